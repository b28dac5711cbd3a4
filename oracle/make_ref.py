"""Places the reference project's own CPU implementation of the expert forward under oracle/_ref/.

    python oracle/make_ref.py [reference root]

`reference.py` (73 lines of pure PyTorch, the file the reference's scripts compare against) is
copied, unmodified, from the reference tree into the git-ignored oracle/_ref/ folder, from where
the benchmark's CPU-baseline leg loads it by path (`cpu_baseline.kind` = "reference").  Where
the reference tree is absent nothing is copied and the benchmark times the CPU restatement in
oracle/experts_oracle.py instead (`kind` = "port").  Nothing under oracle/_ref/ is tracked.
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REL = os.path.join("build", "torch28-cxx11-cu129-x86_64-linux", "yamoe", "reference.py")


def make_ref(root: str = os.environ.get("YAMOE_REFERENCE_ROOT", "/root/reference")) -> str | None:
    src = os.path.join(root, REL)
    if not os.path.exists(src):
        return None
    dst_dir = os.path.join(HERE, "_ref")
    os.makedirs(dst_dir, exist_ok=True)
    dst = os.path.join(dst_dir, "reference.py")
    shutil.copyfile(src, dst)
    return dst


if __name__ == "__main__":
    print(make_ref(*sys.argv[1:2]) or "reference tree not found: nothing copied")
