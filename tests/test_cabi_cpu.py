"""CPU-side checks of the C-ABI library: it loads, exports what include/b200_hstu.h declares,
rejects bad arguments without touching a device, and its host-side mask / block-skipping rule
agree with the oracle."""

import ctypes
import os
import random
import re

import pytest
import torch

from generative_recommenders_b200 import _cabi
from oracle import hstu_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    hdr = open(os.path.join(ROOT, "include", "b200_hstu.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    declared = set(re.findall(r"\b(b200_hstu_[a-z0-9_]+)\s*\(", hdr))
    assert len(declared) >= 16
    lib = ctypes.CDLL(_cabi.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(lib, name), name
    assert declared == set(_cabi.EXPORTS)
    assert _cabi.lib().b200_hstu_version() >= 100


def test_struct_layout_matches_header():
    # the structs are plain C: spot-check the sizes the Python mirror computes
    assert ctypes.sizeof(_cabi.AttnArgs) % 8 == 0
    assert _cabi.AttnArgs.total_L.offset == 8 * 12 + 8 * 16
    # ... delta_size, dropout_ratio, the optional bias gradient, then the dropout seed as the last field
    assert _cabi.AttnArgs.dropout_ratio.offset == _cabi.AttnArgs.delta_size.offset + 4
    assert _cabi.AttnArgs.d_bias_by_distance.offset == ctypes.sizeof(_cabi.AttnArgs) - 16
    assert _cabi.AttnArgs.dropout_seed.offset == ctypes.sizeof(_cabi.AttnArgs) - 8
    assert ctypes.sizeof(_cabi.AttnFp8Args) == ctypes.sizeof(_cabi.AttnArgs) + 32


def test_bad_arguments_are_rejected_on_the_host():
    lib = _cabi.lib()
    assert lib.b200_hstu_attn_fwd(None, None) == -1
    assert b"NULL" in lib.b200_hstu_last_error()
    a = _cabi.AttnArgs()
    a.B, a.H, a.dqk, a.dv, a.total_L, a.max_seq_len = 2, 2, 32, 32, 10, 0
    assert lib.b200_hstu_attn_fwd(a, None) == -1
    assert b"max_seq_len" in lib.b200_hstu_last_error()
    a.max_seq_len = 16
    a.dtype = 7
    assert lib.b200_hstu_attn_fwd(a, None) == -1
    a.dtype = _cabi.F32
    assert lib.b200_hstu_attn_fwd(a, None) == -1  # q is NULL
    # a dropout rate outside [0, 1) is refused on the host, before anything is launched (the pointers
    # below are never followed: validation only asks whether they are NULL)
    a.q = a.k = a.v = a.out = a.seq_offsets = 256
    a.dropout_ratio = 1.0
    assert lib.b200_hstu_attn_fwd(a, None) == -1
    assert b"dropout_ratio" in lib.b200_hstu_last_error()
    a.dropout_ratio = -0.5
    assert lib.b200_hstu_attn_fwd(a, None) == -1
    a.dropout_ratio = 0.0
    a.q = a.k = a.v = a.out = a.seq_offsets = None
    a.B = 0  # an empty batch is a no-op
    assert lib.b200_hstu_attn_fwd(a, None) == 0
    n = _cabi.NormMulArgs()
    n.rows, n.H, n.V, n.act = 4, 2, 8, 5
    assert lib.b200_hstu_norm_mul_fwd(n, None) == -1
    assert lib.b200_hstu_layer_norm_fwd(None, 0, None, None, None, 0, None, None, 4, 0, 1e-5, 0, None) == -1
    assert lib.b200_hstu_layer_norm_bwd_workspace_bytes(512) > 0
    st = (ctypes.c_int32 * 3)(5, 5, 5)
    assert lib.b200_hstu_attn_status_async(None, 0, st, None) == -1
    assert lib.b200_hstu_attn_status_async(a, 3, st, None) == -1
    assert lib.b200_hstu_attn_status_async(a, 0, st, None) == 0 and list(st) == [0, 0, 0]   # no workspace: nothing to read
    assert lib.b200_hstu_selftest_bounded_wait(None, None, None) == -1


def test_host_mask_matches_reference_masks(golden):
    lib = _cabi.lib()
    for c in golden("masks.pt"):
        if c["t"] is None:
            t = 0
        else:
            t = c["t"]
        L = c["L"]
        Lt = c["mask"].shape[0]      # min(L, 24)
        got = torch.tensor([[lib.b200_hstu_host_mask(L, t, 24, c["c"], c["W"], c["F"], i, j) for j in range(Lt)]
                            for i in range(Lt)], dtype=torch.uint8).view(Lt, Lt)
        assert torch.equal(got, c["mask"]), c


def _range(lib, L, t, N, c, W, F, m0, T):
    lo, hi, dg = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
    lib.b200_hstu_host_kv_range(L, t, N, c, W, F, m0, T, ctypes.byref(lo), ctypes.byref(hi), ctypes.byref(dg))
    return lo.value, hi.value, dg.value


@pytest.mark.parametrize("T", [4, 32])
def test_block_skipping_rule_never_drops_a_valid_pair(T):
    lib = _cabi.lib()
    rng = random.Random(1234 + T)
    visited = total = 0
    for _ in range(400):
        N = rng.choice([40, 150])
        L = rng.randint(1, N + (8 if rng.random() < 0.1 else 0))
        c = rng.choice([0, 0, 1, 3, 6])
        t = rng.randint(0, max(0, min(L - 1, 12)))
        W = rng.choice([0, 0, 1, 5, 17, 60])
        F = rng.choice([0, 0, 4]) if W > 0 else 0
        Lt = min(L, N)
        mask = O.valid_attn_mask(Lt, t, True, W, c, F, seq_len=L)  # truncated: max_id from the full length
        for m0 in range(0, Lt, T):
            lo, hi, dg = _range(lib, L, t, N, c, W, F, m0, T)
            rows = mask[m0:m0 + T]
            cols = torch.nonzero(rows.any(dim=0)).flatten().tolist()
            for j in cols:
                assert (lo <= j < hi) or (dg >= 0 and dg <= j < dg + T), (L, t, c, W, F, m0, j, lo, hi, dg)
            # the rule is tight on tile granularity for the regular domain without full-attention tails
            total += (Lt + T - 1) // T
            visited += len({j // T for j in range(lo, hi)} | ({dg // T} if dg >= 0 else set()))
    assert visited < total  # something is skipped


def test_backward_tile_rule_never_drops_a_valid_pair():
    """K/V-stationary backward: every query tile holding a row that sees a column of the kv tile
    must be in the visited set (128-row tiles)."""
    lib = _cabi.lib()
    rng = random.Random(99)
    T = 128
    skipped = 0
    for _ in range(220):
        N = 700
        L = rng.randint(1, N)
        # contextual prefixes inside one tile, ending on a tile boundary and spanning several tiles
        c = rng.choice([0, 0, 2, 7, 127, 128, 130, 260, 400])
        t = rng.randint(0, max(0, min(L - 1, 150)))
        W = rng.choice([0, 0, 3, 100, 130, 300])
        F = rng.choice([0, 0, 40]) if W > 0 else 0
        mask = O.valid_attn_mask(L, t, True, W, c, F)
        ntiles = (L + T - 1) // T
        for kt in range(ntiles):
            lo, n, ex = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
            lib.b200_hstu_host_bwd_q_tiles(L, t, N, c, W, F, kt, ctypes.byref(lo), ctypes.byref(n), ctypes.byref(ex))
            visited = set(range(lo.value, lo.value + n.value)) | ({ex.value} if ex.value >= 0 else set())
            cols = mask[:, kt * T:(kt + 1) * T]
            rows = torch.nonzero(cols.any(dim=1)).flatten().tolist()
            need = {r // T for r in rows}
            assert need <= visited, (L, t, c, W, F, kt, sorted(need), sorted(visited))
            skipped += ntiles - len(visited)
    assert skipped > 0


def test_closed_form_row_and_column_masks_equal_the_exact_mask():
    """The per-row / per-column interval masks of the tensor-core kernels == the reference mask."""
    lib = _cabi.lib()
    rng = random.Random(5)
    checked = 0
    for _ in range(250):
        N = 80
        L = rng.randint(1, N)
        c = rng.choice([0, 0, 1, 3, 6])
        t = rng.randint(0, max(0, min(L - 1, 12)))
        W = rng.choice([0, 0, 1, 5, 17, 60])
        F = rng.choice([0, 0, 4, 9]) if W > 0 else 0
        mask = O.valid_attn_mask(L, t, True, W, c, F)
        for tr in (0, 1):
            got = [[lib.b200_hstu_host_interval_mask(L, t, N, c, W, F, i, j, tr) for j in range(L)] for i in range(L)]
            if got[0][0] == -1:
                assert L - t < c + 1
                continue
            assert torch.equal(torch.tensor(got, dtype=torch.bool), mask), (L, t, c, W, F, tr)
            checked += 1
    assert checked > 300
