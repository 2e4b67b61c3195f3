"""``python -m optimus_lm_b200.kernels [gemm|grouped|attention|all]``: kernel micro-benchmarks."""
import sys

from ..ops import bench_kernels

if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else "all"
    if what in ("gemm", "all"):
        bench_kernels.bench_gemm()
    if what in ("grouped", "all"):
        bench_kernels.bench_grouped()
    if what in ("attention", "all"):
        bench_kernels.bench_attention()
