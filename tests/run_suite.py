"""Run every test file in a process of its own and stop at the first that fails (the layout of test/run_suite.py of the
reference): a file that leaves a process group, an environment variable or a CUDA context behind cannot disturb the next.

    python tests/run_suite.py                 # CPU files (-m "not gpu")
    python tests/run_suite.py --gpu           # GPU files (-m gpu)
"""
import argparse
import glob
import os
import subprocess
import sys
import time


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpu", action="store_true")
    ap.add_argument("--pattern", default="test_*.py")
    ap.add_argument("--timeout", type=int, default=3600, help="seconds per file")
    a = ap.parse_args()
    here = os.path.dirname(os.path.abspath(__file__))
    marker = "gpu" if a.gpu else "not gpu"
    for path in sorted(glob.glob(os.path.join(here, a.pattern))):
        t0 = time.time()
        try:
            rc = subprocess.run([sys.executable, "-m", "pytest", path, "-x", "-q", "-m", marker], cwd=os.path.dirname(here),
                                timeout=a.timeout).returncode
        except subprocess.TimeoutExpired:
            print(f"{os.path.basename(path)}: no exit within {a.timeout} s")
            return 1
        print(f"{os.path.basename(path)}: exit {rc} in {time.time() - t0:.0f} s")
        if rc not in (0, 5):  # 5: no test of the file carries the marker
            return rc
    return 0


if __name__ == "__main__":
    sys.exit(main())
