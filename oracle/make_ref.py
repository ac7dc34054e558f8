"""Place the reference's own CPU implementation of the attention next to the oracle.

    python oracle/make_ref.py [--reference /path/to/generative-recommenders]

TEST / BENCHMARK INFRASTRUCTURE ONLY.  The reference is pure Python on this path, so there is
nothing to compile: the one file that holds its PyTorch attention
(generative_recommenders/ops/pytorch/pt_hstu_attention.py, which needs nothing but torch and the
fbgemm data-movement ops that ``oracle/reference_shims.py`` provides) is copied, unmodified, to
``oracle/_ref/``.  That folder is ignored by git - no reference source enters this repository's
history - but travels with a checkout to wherever the benchmark runs, so that
``bench.py --impl reference`` and the ``cpu_baseline`` of the default run can time the reference
itself (``kind: "reference"``).  Without it they time the restatement in ``oracle/hstu_oracle.py``
(``kind: "port"``).  Nothing in the product imports either.
"""

import argparse
import filecmp
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REL = os.path.join("generative_recommenders", "ops", "pytorch", "pt_hstu_attention.py")


def make_ref(reference: str) -> str:
    src = os.path.join(reference, REL)
    if not os.path.exists(src):
        raise FileNotFoundError(src)
    dst_dir = os.path.join(HERE, "_ref")
    os.makedirs(dst_dir, exist_ok=True)
    dst = os.path.join(dst_dir, "pt_hstu_attention.py")
    if not (os.path.exists(dst) and filecmp.cmp(src, dst, shallow=False)):
        shutil.copyfile(src, dst)
    return dst


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("HSTU_REFERENCE", ""))
    a = ap.parse_args()
    if not a.reference:
        sys.exit("pass --reference /path/to/generative-recommenders")
    print(make_ref(a.reference))
