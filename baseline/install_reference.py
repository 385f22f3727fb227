"""Install the unmodified reference package into the git-ignored baseline/_ref.

    python baseline/install_reference.py [/path/to/reference]

The reference project (WithNucleusAI/mHC-triton) is pure Python: its pure-PyTorch CPU path
(`mhc/_torch_baseline.py`) is what `bench.py --impl reference` times, and its Triton kernels are
what the side arm `bench.py --impl reference_triton` times on a GPU.  Nothing under baseline/_ref is
part of this repository's history or of its product path; `bench.py` falls back to the CPU oracle
under oracle/ when the directory is absent.  Offline: pip is told to use no index and no build
isolation, and the sources are first copied to a temporary directory because the build writes
egg-info next to them.
"""

import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
TARGET = os.path.join(HERE, "_ref")


def install(source: str = "/root/reference") -> bool:
    if not os.path.isdir(os.path.join(source, "src", "mhc")):
        print(f"no reference sources at {source}: nothing installed")
        return False
    if os.path.exists(os.path.join(TARGET, "mhc", "_torch_baseline.py")):
        return True
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "reference")
        shutil.copytree(source, src)
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps", "--quiet",
               "--find-links", "/opt/wheelhouse", "--target", TARGET, src]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            return False
    return True


if __name__ == "__main__":
    ok = install(*sys.argv[1:2])
    print("installed" if ok else "not installed", TARGET)
