"""Device-timed comparison of the four GEMM + all-scatter overlap patterns.

    python examples/benchmark_patterns.py [M N K]
"""

import sys

from tileccl_b200 import benchmarks


def main() -> None:
    M, N, K = (int(x) for x in sys.argv[1:4]) if len(sys.argv) >= 4 else (8192, 4096, 2048)
    print(benchmarks.render(benchmarks.bench_patterns(M=M, N=N, K=K)))


if __name__ == "__main__":
    main()
