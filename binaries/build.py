"""Builds a wheel of the package with the CUDA library inside (reference binaries/build.py builds the pure-Python
wheel; here the build step also runs nvcc through setup.py).

    python binaries/build.py            # dist/pippy_b200-<version>-*.whl
    python binaries/build.py --dry-run  # print the commands only
"""
import argparse
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("--skip-cuda", action="store_true", help="package the Python sources only (PIPPY_B200_SKIP_BUILD=1)")
    args = ap.parse_args()
    env = dict(os.environ)
    if args.skip_cuda:
        env["PIPPY_B200_SKIP_BUILD"] = "1"
    cmds = [[sys.executable, "-m", "pip", "wheel", "--no-deps", "--no-build-isolation", "-w", "dist", ROOT]]
    for cmd in cmds:
        print("+", " ".join(cmd))
        if not args.dry_run:
            rc = subprocess.call(cmd, cwd=ROOT, env=env)
            if rc:
                return rc
    return 0


if __name__ == "__main__":
    sys.exit(main())
