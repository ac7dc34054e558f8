"""Print the in-kernel timeline of CTA 0 of an attention launch.

    B200_HSTU_TRACE_BUILD=1 python generative-recommenders_b200/build.py --force    # marks compiled in
    python generative-recommenders_b200/trace_timeline.py [--launch fwd|dkdv|dq] [--workload config1|long]
    python generative-recommenders_b200/build.py --force                            # back to the normal build

A profiling aid, not part of the product path: with the marks compiled in, the roles of CTA 0
(producer, MMA issuer, activation, epilogue) write a clock value and a tag at the points named
below into spare room behind the work lists, and this script prints them merged by time with the
cycles since the role's previous mark.  The marks cost about a hundred cycles each, so the numbers
say where a role waits and in which order things happen, not how fast the normal build is.

Tags, forward (csrc/attn_fwd_sm100.cu): producer 1 item start, 2 Q slot free, 3 K slot free, 4 V slot
free; MMA 10 item start, 11 first scores issued, 12/13 waiting for P of tile A/B, 14/15 P arrived,
20 V arrived, 16/17 next K waited for / arrived, 18/19 next scores of A/B issued, 21 next item's
first scores issued; activation 30 tile start, 31 scores arrived, 32 scores in registers, 37
P stored, 33 P handed over.
Backward (csrc/attn_bwd_sm100.cu): producer 1-4 as above for the stationary and streamed tiles; MMA 10
item start, 12/14 waiting for / got P, 16 after dV += P^T dO, 13/15 waiting for / got dS, 17 after
the dK | dQ product; activation 30/31 waiting for / got the scores, 37 phase A done, 33 P handed over,
32 dP arrived, 34 dS handed over; epilogue 40 item start, 41 accumulator complete, 42 stored.
"""

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--launch", choices=["fwd", "dkdv", "dq"], default="fwd")
    ap.add_argument("--workload", choices=["config1", "long"], default="config1",
                    help="config1: the benchmark batch; long: 160 sequences of 4096 tokens, one head")
    ap.add_argument("--limit", type=int, default=400, help="print at most this many records")
    args = ap.parse_args()
    os.environ["B200_HSTU_TRACE"] = {"fwd": "1", "dkdv": "dkdv", "dq": "dq"}[args.launch]

    import importlib
    pkg = importlib.import_module("generative-recommenders_b200")
    _cabi, W = pkg._cabi, importlib.import_module("generative-recommenders_b200.workloads")
    HA = importlib.import_module("generative-recommenders_b200.hstu_attention")

    dev = "cuda:0"
    if args.workload == "config1":
        w = W.config1()
        q, k, v = w.qkv(device=dev)
        offs, nt = w.seq_offsets.to(torch.int32).to(dev), w.num_targets.to(torch.int32).to(dev)
        N, alpha = w.max_seq_len, w.alpha
    else:
        B, L, H, N = 160, 4096, 1, 4096
        g = torch.Generator().manual_seed(0)
        q, k, v = ((torch.randn(B * L, H, 128, generator=g) * 0.5).bfloat16().to(dev) for _ in range(3))
        offs, nt, alpha = (torch.arange(B + 1) * L).to(torch.int32).to(dev), None, 1.0 / 128
    a = _cabi.AttnArgs()
    HA._fill_common(a, q, k, v, offs, nt, None, N, alpha, 0, 0, 0, None)
    out = torch.empty_like(v)
    keep = [out]
    if args.launch == "fwd":
        a.out, a.o_row_stride, a.o_head_stride = out.data_ptr(), out.stride(0), out.stride(1)
        call, which = _cabi.lib().b200_hstu_attn_fwd, 0
    else:
        dout, dq, dk, dv = (torch.randn_like(v) if i == 0 else torch.empty_like(v) for i in range(4))
        keep += [dout, dq, dk, dv]
        a.dout, a.dq, a.dk, a.dv_ = dout.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
        for name, t in (("do", dout), ("dq", dq), ("dk", dk), ("dv", dv)):
            setattr(a, name + "_row_stride", t.stride(0))
            setattr(a, name + "_head_stride", t.stride(1))
        call, which = _cabi.lib().b200_hstu_attn_bwd, 1
    need = _cabi.lib().b200_hstu_attn_workspace_bytes(a, which)
    records, roles = 1024, 4
    room = roles * records * 16
    ws = torch.zeros(need + room, dtype=torch.uint8, device=dev)
    a.workspace, a.workspace_bytes = ws.data_ptr(), need + room
    for _ in range(3):
        ws[need:].zero_()
        _cabi.check(call(a, torch.cuda.current_stream().cuda_stream), "traced launch")
        torch.cuda.synchronize()
    tr = ws[need:].view(torch.int64).view(roles, records, 2).cpu()
    names = ["producer", "mma", "act", "act1" if args.launch == "fwd" else "epilogue"]
    ev = [(int(tr[r, i, 0]), names[r], int(tr[r, i, 1])) for r in range(roles) for i in range(records)
          if tr[r, i, 0] > 0 and tr[r, i, 1] < 1000]
    if not ev:
        print("no records: is the library built with B200_HSTU_TRACE_BUILD=1?")
        return 1
    ev.sort()
    t0, last = ev[0][0], {}
    print("%d records, %d cycles from the first to the last" % (len(ev), ev[-1][0] - t0))
    for t, name, tag in ev[:args.limit]:
        print("%9d  %-8s %3d  (+%d)" % (t - t0, name, tag, t - last.get(name, t0)))
        last[name] = t
    return 0


if __name__ == "__main__":
    sys.exit(main())
