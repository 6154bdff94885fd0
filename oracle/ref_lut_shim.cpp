// C entry points around the reference project's own LUT helper headers
// (csrc/lut8_unsigned.cuh and csrc/lut8.cuh compile as plain C++).  The headers are
// found through -I at build time; nothing from them is stored in this repository.
// Used only by tests to check the oracle's table arithmetic against the real thing.
#include "lut8_unsigned.cuh"
#include "lut8.cuh"

extern "C" {

// Full 256-entry unsigned subset-sum table, built the way a warp does: lane by lane.
void ref_build_unsigned_table(float* table, const float* values) {
  for (unsigned lane = 0; lane < 32; ++lane)
    fluxbin_w3_lut::build_lane_unsigned(table, values, lane);
}

// Full 256-entry signed (+/-) table.
void ref_build_signed_table(float* table, const float* values) {
  for (unsigned lane = 0; lane < 32; ++lane) fluxbin_lut::build_lane(table, values, lane);
}

// One base's eight sign bits out of sixteen interleaved bits.
unsigned ref_pattern(unsigned word) { return fluxbin_lut::pattern(word); }
}
