"""Convenience runner (the reference ships tests/run_tests.py): CPU suite, then the packer
comparison printed as a table. ``python tests/run_tests.py [--gpu]``"""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def main() -> int:
    marker = "gpu" if "--gpu" in sys.argv else "not gpu"
    rc = subprocess.call([sys.executable, "-m", "pytest", os.path.join(ROOT, "tests"), "-q", "-m", marker], cwd=ROOT)
    sys.path.insert(0, ROOT)
    import numpy as np
    from mini_trainer_b200.data import packer as P
    rng = np.random.default_rng(42)
    kinds = rng.choice(4, 500, p=[0.5, 0.3, 0.15, 0.05])
    lengths = rng.integers(np.array([100, 2000, 20000, 60000])[kinds], np.array([2000, 20000, 60000, 100000])[kinds]).tolist()
    lpt = P.packing_stats(lengths, P.lpt_pack_all(lengths, 130000, 8), 130000)
    greedy = P.packing_stats(lengths, [P.batch_lengths_to_minibatches(lengths, 130000, 8, r) for r in range(8)], 130000)
    print(f"{'packer':>8} {'minibatches':>12} {'avg balance':>12} {'worst':>8} {'row eff':>8}")
    for name, s in (("LPT", lpt), ("greedy", greedy)):
        print(f"{name:>8} {s['num_minibatches']:>12} {s['avg_balance']:>12.3f} {s['worst_balance']:>8.3f} {s['row_efficiency']:>8.3f}")
    return rc


if __name__ == "__main__":
    sys.exit(main())
