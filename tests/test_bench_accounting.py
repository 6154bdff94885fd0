"""The byte counts the benchmark divides by: they must be the algorithmic bytes of the path
(packed planes, scales, zero points, activations in and out), not anything measured."""
import importlib.util
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_w3_bytes_match_the_published_accounting():
    bench = load_bench()
    # planes 3OK/8, fp16 scales 2GO, x 2K, y 2O, and zero points as stored (uint8) or as fp16
    for (o, k), with_fp16_zeros in (((4096, 4096), 6_832_128), ((1024, 4096), 1_714_176),
                                    ((12288, 4096), 20_480_000), ((4096, 12288), 20_480_000)):
        groups = k // 128
        stored = bench.gemv_bytes(o, k)
        assert stored == 3 * o * k // 8 + 2 * groups * o + groups * o + 2 * k + 2 * o
        assert stored + groups * o == with_fp16_zeros
    layer = sum(bench.gemv_bytes(o, k) + (k // 128) * o for _, o, k in bench.SHAPES)
    assert layer == 78_532_608  # per layer, zero points as fp16


def test_binary_basis_bytes_match_the_published_accounting():
    bench = load_bench()
    assert bench.bb_bytes(4096, 4096) == 4_505_728
    assert bench.bb_bytes(1024, 4096) == 1_144_960
    assert bench.bb_bytes(12288, 4096) == 13_467_776
    assert bench.bb_bytes(4096, 12288) == 12_943_488
