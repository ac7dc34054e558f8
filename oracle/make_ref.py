"""Place the reference's own CPU implementation of the attention next to the oracle.

    python oracle/make_ref.py [--reference /path/to/generative-recommenders]

TEST / BENCHMARK INFRASTRUCTURE ONLY.  The reference is pure Python on this path, so there is
nothing to compile: the file that holds its PyTorch attention
(generative_recommenders/ops/pytorch/pt_hstu_attention.py, which needs nothing but torch and the
fbgemm data-movement ops that ``oracle/reference_shims.py`` provides) is copied, unmodified, to
``oracle/_ref/``, and so are the few files its Triton forward kernel lives in
(ops/triton/triton_hstu_attention.py with ops/triton/triton_attention_utils.py, ops/utils.py and
common.py), under their package paths.  That folder is ignored by git - no reference source
enters this repository's history - but travels with a checkout to wherever the benchmark runs,
so that ``bench.py --impl reference`` and the ``cpu_baseline`` of the default run can time the
reference itself (``kind: "reference"``), and the default run can time the reference's own GPU
paths next to this library's.  Without it the CPU legs time the restatement in
``oracle/hstu_oracle.py`` (``kind: "port"``).  Nothing in the product imports either.
"""

import argparse
import filecmp
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REL = os.path.join("generative_recommenders", "ops", "pytorch", "pt_hstu_attention.py")
# the package files the Triton forward needs, copied under their package paths
TREE = [
    "generative_recommenders/__init__.py",
    "generative_recommenders/common.py",
    "generative_recommenders/ops/__init__.py",
    "generative_recommenders/ops/utils.py",
    "generative_recommenders/ops/pytorch/__init__.py",
    "generative_recommenders/ops/pytorch/pt_hstu_attention.py",
    "generative_recommenders/ops/triton/__init__.py",
    "generative_recommenders/ops/triton/triton_attention_utils.py",
    "generative_recommenders/ops/triton/triton_hstu_attention.py",
]


def _copy(src, dst):
    os.makedirs(os.path.dirname(dst), exist_ok=True)
    if not (os.path.exists(dst) and filecmp.cmp(src, dst, shallow=False)):
        shutil.copyfile(src, dst)


def make_ref(reference: str) -> str:
    src = os.path.join(reference, REL)
    if not os.path.exists(src):
        raise FileNotFoundError(src)
    dst_dir = os.path.join(HERE, "_ref")
    dst = os.path.join(dst_dir, "pt_hstu_attention.py")
    _copy(src, dst)
    for rel in TREE:
        s_ = os.path.join(reference, *rel.split("/"))
        d_ = os.path.join(dst_dir, *rel.split("/"))
        if os.path.exists(s_):
            _copy(s_, d_)
        elif rel.endswith("__init__.py"):   # a namespace package in the reference: an empty marker will do
            os.makedirs(os.path.dirname(d_), exist_ok=True)
            open(d_, "a").close()
    return dst


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("HSTU_REFERENCE", ""))
    a = ap.parse_args()
    if not a.reference:
        sys.exit("pass --reference /path/to/generative-recommenders")
    print(make_ref(a.reference))
