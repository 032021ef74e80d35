"""Range profiler: runs the range everywhere; lists kernels by name on a GPU."""
import pytest
import torch

from pegainfer_b200.utils.range_profiler import RangeProfiler


def test_range_runs_without_a_gpu_and_reports_unavailable():
    if torch.cuda.is_available():
        pytest.skip("CPU behaviour")
    hit = []
    with RangeProfiler("cpu range") as rp:
        hit.append(1)
    assert hit == [1] and not rp.available and rp.kernels() == []
    assert "not available" in rp.report()
    assert rp.sol(bytes_moved=1e9, peak_gbs=1000.0) == {"span_us": 0.0, "kernel_us": 0.0}


@pytest.mark.gpu
def test_kernels_of_a_range_by_name_on_gpu():
    from pegainfer_b200.ops import cuda as K

    x = torch.randn(64, 4096, device="cuda:0").bfloat16()
    w = torch.randn(4096, 4096, device="cuda:0").bfloat16() * 0.02
    nw = torch.ones(4096, device="cuda:0").bfloat16()
    K.linear(x, w)
    K.rms_norm(x, nw, 1e-6)
    torch.cuda.synchronize()
    with RangeProfiler("two ops") as rp:
        for _ in range(3):
            K.linear(x, w)
        K.rms_norm(x, nw, 1e-6)
    assert rp.available
    rows = rp.kernels()
    names = " ".join(r.name for r in rows)
    assert "gemm" in names and "rms_norm" in names, names
    gemm = [r for r in rows if "gemm" in r.name][0]
    assert gemm.launches == 3 and 0 < gemm.min_us <= gemm.mean_us <= gemm.max_us
    s = rp.sol(bytes_moved=3 * 4096 * 4096 * 2, peak_gbs=6500.0)
    assert s["span_us"] > 0 and 0 < s["frac_of_copy_peak"] < 1.5
    assert "launches" in rp.report()
