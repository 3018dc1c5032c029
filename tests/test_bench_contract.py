"""Host-side checks of the benchmark harness that need no GPU."""
import importlib.util
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def _bench():
    spec = importlib.util.spec_from_file_location("heirloom_bench", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_the_recorded_gemm_traffic_belongs_to_the_current_gemm_source():
    """`roofline.traffic` comes from an ncu capture; the capture is only valid for the kernel source it ran with."""
    traffic, note = _bench().gemm_traffic()
    assert traffic is not None and traffic > 0, note


def test_flops_per_token_of_the_benchmark_shape():
    b = _bench()
    # 6 * (12 * (4*768^2 + 2*768*3072) + 768*50304) + 6 * 12 * 1024 * 768
    assert b.flops_per_token(b.GPT) == 798031872.0
