"""Device-vs-host correctness harness (the reference's crates/axonml-core/examples/gpu_test.rs):
runs this package's kernels against the C++ host oracle over sizes 1..4096 and prints the report.
Without a GPU it reports that no device was found and exits 0.

    python examples/gpu_test.py
"""
import torch

from axonml_b200.core import gpu_tests


def main() -> int:
    if not torch.cuda.is_available():
        print("no CUDA device: nothing to compare against the host oracle")
        return 0
    report = gpu_tests.run_all_tests()
    report.print_summary()
    return 0 if report.all_passed() else 1


if __name__ == "__main__":
    raise SystemExit(main())
