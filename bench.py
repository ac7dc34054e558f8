"""Benchmark of the HSTU jagged-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload config1|config3]

A step is one forward + backward of ``hstu_mha`` over one synthetic batch with the shapes of the
benchmark configuration (bf16, B=64 sequences per GPU, L ~ U{128..1024}, N=1024, H=4, d=128,
targets ~ U{1..32}).  With N > 1 (launched by torchrun, one rank per GPU) the batch has 64*N
sequences split over the ranks by token count; there is no collective on the data path, the
only collectives are the barrier / max-reduction used for timing.

One JSON line is printed by rank 0.  ``value`` is whole-job TFLOP/s of forward + backward counted
with the nominal causal formula 3.5 * 4*H*d*sum(L^2)/2, measured with CUDA events with the
inputs resident in HBM.  ``e2e`` is the same metric through the public ``hstu_mha`` with pinned
host tensors copied in and results copied out inside the timed region, every step (upload,
compute and download run on three streams, so consecutive steps overlap).  ``roofline`` describes
the dominant kernel, ``cpu_baseline`` the CPU oracle timed on the host cores on a bounded
sample.
"""

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
SEQS_PER_GPU = 64


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.005)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(1.0)

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def make_workload(world, name):
    from generative_recommenders_b200 import workloads as W

    if name in ("config3", "config3_fp8"):
        return W.config3(256 * world)
    return W.config1(SEQS_PER_GPU * world)


def rank_shard(w, rank, world):
    from generative_recommenders_b200 import sharding, workloads as W

    if world == 1:
        return w
    bins = sharding.partition_by_tokens(w.lengths.tolist(), world)
    sub = W.subset(w, bins[rank])
    sub.seed = w.seed + 17 * rank
    return sub


def pin_rank_to_cores(local_rank, world):
    """Give every rank of a multi-GPU run its own share of the host cores (the step is a few
    hundred microseconds long: a launching thread that migrates, or shares a core with another
    rank's sampler thread, shows up as idle time on its GPU).  Returns the cores, or None."""
    try:
        cores = sorted(os.sched_getaffinity(0))
        if world <= 1 or len(cores) < 2 * world:
            return None
        per = len(cores) // world
        mine = cores[local_rank * per:(local_rank + 1) * per]
        os.sched_setaffinity(0, mine)
        torch.set_num_threads(max(1, min(per, 8)))
        return mine
    except Exception:
        return None


def dist_stats(x, _unused=None):
    """min / max / mean over steps of a list of per-step milliseconds."""
    s = sorted(x)
    n = len(s)
    return {"median": round(s[n // 2], 5), "min": round(s[0], 5), "p90": round(s[min(n - 1, (9 * n) // 10)], 5),
            "mean": round(sum(s) / n, 5), "n": n}


def capture_step(step, inputs, dev):
    """One forward + backward of the public API captured into a CUDA graph; replaying it launches
    the same kernels with no host work in between.  Returns (graph, outputs) or (None, None)."""
    try:
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                step(*inputs)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            res = step(*inputs)
        return graph, res
    except Exception as ex:  # pragma: no cover - depends on the driver
        sys.stderr.write("bench: CUDA graph capture of the step failed (%s); timing eager launches\n" % ex)
        torch.cuda.synchronize()
        return None, None


def run_ours(args):
    import generative_recommenders_b200 as G
    from generative_recommenders_b200 import _cabi

    world, rank, local_rank, dev, dist = _dist_setup()
    cores = pin_rank_to_cores(local_rank, world)
    w_all = make_workload(world, args.workload)
    w = rank_shard(w_all, rank, world)
    fwd_only = args.workload == "config3" or args.fwd_only
    N, alpha = w.max_seq_len, w.alpha
    q, k, v, do = w.qkv(device="cpu", with_dout=True)
    hq, hk, hv, hdo = (t.pin_memory() for t in (q, k, v, do))
    offs = w.seq_offsets.to(torch.int32).to(dev)
    nt = None if w.num_targets is None else w.num_targets.to(torch.int32).to(dev)
    dq_, dk_, dv_, ddo = (t.to(dev) for t in (q, k, v, do))
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    kw = dict(num_targets=nt, max_attn_len=w.max_attn_len, contextual_seq_len=w.contextual_seq_len)

    def step(qd, kd, vd, dod):
        if fwd_only:
            with torch.no_grad():
                return G.hstu_mha(N, alpha, qd, kd, vd, offs, **kw), None
        qd.requires_grad_(True); kd.requires_grad_(True); vd.requires_grad_(True)
        qd.grad = kd.grad = vd.grad = None
        out = G.hstu_mha(N, alpha, qd, kd, vd, offs, **kw)
        out.backward(dod)
        return out, (qd.grad, kd.grad, vd.grad)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step(dq_, dk_, dv_, ddo)
    barrier()

    # ---- device-resident timing.  A step is one forward + backward through the public API; it is
    # captured once into a CUDA graph and replayed, so that the timed region holds the kernels and
    # nothing of the host (eager launches of a 0.2 ms step are bound by the Python / autograd
    # dispatch of the slowest rank; they are timed further down and reported next to this).
    # Per-step CUDA events, L2 flushed (untimed) between steps; --steps K is repeated for as many
    # rounds as it takes to fill half a second, every step of every round is timed.
    graph = None
    if not args.eager:
        graph, _ = capture_step(step, (dq_.detach().clone(), dk_.detach().clone(), dv_.detach().clone(), ddo), dev)
    run = graph.replay if graph is not None else (lambda: step(dq_, dk_, dv_, ddo))
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    run()
    torch.cuda.synchronize()
    est_ms = max(1e-3, (time.perf_counter() - t0) * 1e3)
    rounds = int(max(1, min(400, -(-500.0 // (args.steps * est_ms))))) if args.rounds <= 0 else args.rounds
    if dist is not None:   # every rank times the same number of steps
        r_ = torch.tensor([rounds], device=dev)
        dist.all_reduce(r_, op=dist.ReduceOp.MAX)
        rounds = int(r_.item())
    n_timed = rounds * args.steps
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_timed)]
    launches0 = _cabi.launch_count()
    with ClockSampler(local_rank) as clocks:
        barrier()
        for s, e in ev:
            flush.zero_()
            s.record()
            run()
            e.record()
        barrier()
    launches = _cabi.launch_count() - launches0
    step_ms = [s.elapsed_time(e) for s, e in ev]
    ms_total = sum(step_ms)
    launches_per_step = 2 if fwd_only else 4   # planning + forward (+ the two backward launches)
    if graph is not None:
        launches = launches_per_step * n_timed   # replayed launches are not seen by the library's counter

    # ---- eager launches: forward / backward separately, with the library's per-kernel event timing
    # switched on (CUDA events recorded by the library around each kernel on the launch stream)
    _cabi.profile_enable(True)
    fe = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
          for _ in range(max(20, min(args.steps, 100)))]
    for a, b, c in fe:
        flush.zero_()
        qd = dq_.detach().requires_grad_(not fwd_only); kd = dk_.detach().requires_grad_(not fwd_only)
        vd = dv_.detach().requires_grad_(not fwd_only)
        a.record()
        if fwd_only:
            with torch.no_grad():
                out = G.hstu_mha(N, alpha, qd, kd, vd, offs, **kw)
            b.record()
        else:
            out = G.hstu_mha(N, alpha, qd, kd, vd, offs, **kw)
            b.record()
            out.backward(ddo)
        c.record()
    torch.cuda.synchronize()
    fwd_ms = sorted(a.elapsed_time(b) for a, b, c in fe)[len(fe) // 2]
    bwd_ms = sorted(b.elapsed_time(c) for a, b, c in fe)[len(fe) // 2]
    eager_ms = sorted(a.elapsed_time(c) for a, b, c in fe)[len(fe) // 2]
    kernel_ms, kernel_stats = {}, {}
    for kind in ("plan", "attn_fwd", "attn_bwd_dkdv", "attn_bwd_dq"):
        vals = _cabi.profile_collect(kind)
        if vals:
            kernel_ms[kind] = sum(vals) / len(vals)
            kernel_stats[kind] = dist_stats(vals, None)
    _cabi.profile_enable(False)

    # ---- end to end through the public API from pinned host memory.  Every step copies its inputs
    # host -> device and its results device -> host; the three parts run on three streams (upload,
    # compute, download) with double-buffered device inputs, so that step i + 1 uploads while step i
    # computes and step i - 1 downloads - the way an input pipeline feeds a training loop.
    e2e_steps = max(3, min(args.steps, 20))
    res_host = [torch.empty_like(t).pin_memory() for t in ((q,) if fwd_only else (q, q, k, v))]
    host_in = [hq, hk, hv] + ([] if fwd_only else [hdo])
    dev_in = [[torch.empty_like(t, device=dev) for t in host_in] for _ in range(2)]
    s_comp = torch.cuda.current_stream(dev)
    s_up, s_down = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    computed = [None, None]     # event: the step that read dev_in[slot] has finished
    state = {"i": 0, "last_down": None}

    def e2e_step():
        i = state["i"]
        slot = i & 1
        with torch.cuda.stream(s_up):
            if computed[slot] is not None:
                s_up.wait_event(computed[slot])
            for dst, src in zip(dev_in[slot], host_in):
                dst.copy_(src, non_blocking=True)
            uploaded = torch.cuda.Event()
            uploaded.record(s_up)
        s_comp.wait_event(uploaded)
        bufs = [t.detach() for t in dev_in[slot]]   # fresh aliases: step() marks its inputs as leaves
        out, grads = step(bufs[0], bufs[1], bufs[2], None if fwd_only else bufs[3])
        done = torch.cuda.Event()
        done.record(s_comp)
        computed[slot] = done
        results = [out] + (list(grads) if grads is not None else [])
        with torch.cuda.stream(s_down):
            s_down.wait_event(done)
            for dst, g_ in zip(res_host, results):
                g_.record_stream(s_down)
                dst.copy_(g_, non_blocking=True)
            fin = torch.cuda.Event()
            fin.record(s_down)
        state["last_down"] = fin
        state["i"] = i + 1

    def e2e_drain():
        if state["last_down"] is not None:
            s_comp.wait_event(state["last_down"])

    e2e_step()
    e2e_drain()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_drain()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    elem = q.element_size()
    h2d = sum(t.numel() for t in ((q, k, v) if fwd_only else (q, k, v, do))) * elem
    d2h = sum(t.numel() for t in res_host) * elem

    # ---- validation across ranks: every rank hands the rows of one of its sequences (inputs and
    # the output it computed) to rank 0, which runs those sequences again as one batch on its own GPU;
    # a sequence's rows do not depend on what else is in the batch, so the bits must agree.  This
    # gather is the only collective that touches data, and it is outside every timed region.
    validated = None
    with torch.no_grad():
        mine_out = G.hstu_mha(N, alpha, dq_.detach(), dk_.detach(), dv_.detach(), offs, **kw)
        pick = int(torch.argmax(w.lengths))    # this rank's longest sequence
        lo_, hi_ = int(w.seq_offsets[pick]), int(w.seq_offsets[pick + 1])
        pack = torch.zeros((4, N) + tuple(q.shape[1:]), dtype=q.dtype, device=dev)
        for i_, t_ in enumerate((dq_, dk_, dv_, mine_out)):
            pack[i_, :hi_ - lo_] = t_.detach()[lo_:hi_]
        meta = torch.tensor([hi_ - lo_, 0 if w.num_targets is None else int(w.num_targets[pick])], dtype=torch.int64, device=dev)
        if dist is not None:
            packs = [torch.empty_like(pack) for _ in range(world)]
            metas = [torch.empty_like(meta) for _ in range(world)]
            dist.all_gather(packs, pack)
            dist.all_gather(metas, meta)
        else:
            packs, metas = [pack], [meta]
        if rank == 0:
            lens = torch.stack(metas)[:, 0].cpu()
            vo = torch.cat([lens.new_zeros(1), torch.cumsum(lens, 0)]).to(torch.int32).to(dev)
            vnt = None if w.num_targets is None else torch.stack(metas)[:, 1].to(torch.int32).to(dev)
            cat = [torch.cat([p_[i_, :int(n_)] for p_, n_ in zip(packs, lens)]) for i_ in range(4)]
            again = G.hstu_mha(N, alpha, cat[0], cat[1], cat[2], vo, num_targets=vnt, max_attn_len=w.max_attn_len,
                               contextual_seq_len=w.contextual_seq_len)
            torch.cuda.synchronize()
            validated = {"ok": bool(torch.equal(again, cat[3])), "sequences": int(world), "rows": int(lens.sum()),
                         "how": "rows of one sequence per rank gathered%s and recomputed on rank 0: bit-identical" %
                                (" over NCCL" if dist is not None else "")}

    # ---- reduce over ranks: time = max, work = sum
    # FLOP count: the reference bench's causal formula 4*H*d*sum(L^2)/2; with a local window that
    # formula counts pairs the mask removes (configs[3]: 4x too many), so such workloads count the
    # exact number of visible (q, k) pairs instead and say so in the metric name
    use_exact = w.max_attn_len > 0
    flops_fwd = 4.0 * w.num_heads * w.attn_dim * w.exact_pairs() if use_exact else w.causal_flops_fwd()
    mult = 1.0 if fwd_only else 3.5
    lsq = float((w.lengths.double() ** 2).sum())
    mine = torch.tensor([ms_total / n_timed, e2e_ms, fwd_ms, bwd_ms, eager_ms, kernel_ms.get("plan", 0.0),
                         kernel_ms.get("attn_fwd", 0.0), kernel_ms.get("attn_bwd_dkdv", 0.0),
                         kernel_ms.get("attn_bwd_dq", 0.0), float(w.total_tokens), lsq, flops_fwd, float(launches)],
                        dtype=torch.float64, device=dev)
    if dist is not None:
        allr = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allr, mine)
        allr = torch.stack(allr).cpu()
    else:
        allr = mine.cpu().view(1, -1)
    ms_per_step, e2e_ms, fwd_ms_max, bwd_ms_max = (float(allr[:, i_].max()) for i_ in range(4))
    flops_fwd_all, tokens_all, launches_all = float(allr[:, 11].sum()), float(allr[:, 9].sum()), float(allr[:, 12].sum())
    value = mult * flops_fwd_all / (ms_per_step * 1e-3) / 1e12
    e2e_value = mult * flops_fwd_all / (e2e_ms * 1e-3) / 1e12
    fields = ["step_ms", "e2e_ms", "fwd_ms_eager", "bwd_ms_eager", "step_ms_eager", "plan_kernel_ms", "fwd_kernel_ms",
              "dkdv_kernel_ms", "dq_kernel_ms", "tokens", "sum_L2"]
    ranks = {f_: {"min": round(float(allr[:, i_].min()), 5), "max": round(float(allr[:, i_].max()), 5),
                  "argmax": int(allr[:, i_].argmax())} for i_, f_ in enumerate(fields)}

    peaks, peak_kind = load_peaks()
    # dominant kernel of the step and its roofline (rank 0's share of the work).  Algorithmic FLOPs
    # per launch with F = 4*H*d*sum(L^2)/2: forward F (two GEMMs); backward dK/dV kernel 2F (S^T, dP^T,
    # dV, dK); backward dQ kernel 0.5F (the dQ GEMM; its recomputation of S and dP is overhead of the
    # two-kernel design and is not counted).
    exact_fwd = 4.0 * w.num_heads * w.attn_dim * w.exact_pairs()
    algo = {"attn_fwd": 1.0, "attn_bwd_dkdv": 2.0, "attn_bwd_dq": 0.5}
    names = {"attn_fwd": "hstu_attn_fwd_sm100_kernel", "attn_bwd_dkdv": "hstu_attn_bwd_sm100_kernel<DKDV=true>",
             "attn_bwd_dq": "hstu_attn_bwd_sm100_kernel<DKDV=false>"}
    cand = {k_: v_ for k_, v_ in kernel_ms.items() if k_ in algo}
    if cand:
        dom = max(cand, key=cand.get)
        dom_ms, dom_flops, dom_name = cand[dom], algo[dom] * flops_fwd, names[dom]
    else:  # CUDA-core path (no per-kernel events): fall back to the step halves
        dom_name, dom_ms, dom_flops = ("attention forward", fwd_ms, flops_fwd) if (fwd_only or fwd_ms >= bwd_ms) \
            else ("attention backward", bwd_ms, 2.5 * flops_fwd)
    ach = dom_flops / (dom_ms * 1e-3) / 1e12
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "dram_traffic.json")
    if os.path.exists(tpath):
        try:
            traffic = json.load(open(tpath)).get(dom_name, {}).get(w.name)
        except Exception:
            traffic = None
    csum = clocks.summary()
    mhz = csum.get("sm_mhz") or 0
    per_kernel = {}
    for k_ in algo:
        if k_ in kernel_ms:
            tf = algo[k_] * flops_fwd / (kernel_ms[k_] * 1e-3) / 1e12
            per_kernel[k_] = {"ms": kernel_stats[k_], "algorithmic_tflops": round(tf, 1),
                              "frac": round(tf / peaks["bf16_tflops"], 4),
                              "frac_sustained": round(tf / peaks["bf16_tflops_sustained"], 4),
                              "ms_x_mhz": round(kernel_stats[k_]["median"] * mhz, 2)}
    if not fwd_only and "attn_bwd_dkdv" in kernel_ms and "attn_bwd_dq" in kernel_ms:
        tb = 2.5 * flops_fwd / ((kernel_ms["attn_bwd_dkdv"] + kernel_ms["attn_bwd_dq"]) * 1e-3) / 1e12
        per_kernel["backward_both_launches"] = {"algorithmic_tflops": round(tb, 1), "frac": round(tb / peaks["bf16_tflops"], 4),
                                                "frac_sustained": round(tb / peaks["bf16_tflops_sustained"], 4)}
    roofline = {"kernel": dom_name, "bound": "tensor", "achieved": round(ach, 2), "peak": peaks["bf16_tflops"],
                "unit": "TFLOP/s", "frac": round(ach / peaks["bf16_tflops"], 4), "traffic": traffic,
                "frac_sustained": round(ach / peaks["bf16_tflops_sustained"], 4),
                "peak_source": peak_kind + " (cuBLAS bf16 burst; frac_sustained: the seconds-long loop under the power cap)",
                "launch_ms": round(dom_ms, 4), "flops_per_launch": dom_flops,
                "flops_model": ("F = 4*H*d*(visible (q,k) pairs)" if use_exact else "nominal causal F = 4*H*d*sum(L^2)/2") +
                               "; fwd F, bwd dK/dV kernel 2F, bwd dQ kernel 0.5F",
                "kernel_ms": {k_: round(v_, 4) for k_, v_ in kernel_ms.items()}, "kernels": per_kernel}

    # ---- further records on the same line: the other configurations and the stage kernels
    blocks = {}
    if args.blocks != "none" and args.workload == "config1" and not args.fwd_only:
        del dev_in, res_host, flush, ev
        torch.cuda.empty_cache()
        if world == 1:
            blocks["reference_gpu"] = block_reference_gpu(dev, w, args)
            torch.cuda.empty_cache()
            blocks["config3"] = block_config3(dev, peaks, args)
            blocks["stages"] = block_stages(dev, peaks, args)
        blocks["config4"] = block_config4(world, rank, dev, dist, args)

    if rank == 0:
        out = {
            "metric": "hstu_mha_%s_tflops%s" % ("fwd" if fwd_only else "fwd_bwd", "_exact_pairs" if use_exact else ""),
            "value": round(value, 3), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "configs[%s]: hstu_mha %s, B=%d seqs/GPU, H=%d, d=%d, N=%d, targets, bf16" % (
                "3" if args.workload == "config3" else "1", "fwd" if fwd_only else "fwd+bwd", len(w.lengths), w.num_heads, w.attn_dim, N),
                "global_batch": len(w_all.lengths), "tokens": int(tokens_all), "seq_len": N,
                "parallelism": "sequence-sharded x%d by token count, no collective" % world,
                "l2": "256 MiB memset between timed steps (untimed)",
                "launch": ("one CUDA graph per step (forward + backward of hstu_mha captured through the public API), replayed"
                           if graph is not None else "eager launches through the public API"),
                "timed_steps": "%d rounds x %d steps, every step timed with its own CUDA events" % (rounds, args.steps),
                "host_cores_per_rank": None if cores is None else len(cores)},
            "step_ms": dist_stats(step_ms, None),
            "step_ms_eager": round(eager_ms, 5),
            "tokens_per_s": round(tokens_all / (ms_per_step * 1e-3), 1),
            "fwd_tflops": round(flops_fwd / (fwd_ms * 1e-3) / 1e12, 2),
            "fwd_ms": round(fwd_ms, 4), "bwd_ms": round(bwd_ms, 4),
            "fwd_tflops_exact_pairs": round(exact_fwd / (fwd_ms * 1e-3) / 1e12, 2),
            "frac_of_nominal_bf16_peak_2250": round(value / world / 2250.0, 4),
            "e2e": {"value": round(e2e_value, 3), "unit": "TFLOP/s", "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d2h), "ms_per_step": round(e2e_ms, 4)},
            "gpu_launches": int(launches_all),
            "clocks": csum,
            "roofline": roofline,
            "ranks": ranks,
            "validated": validated,
        }
        out.update(blocks)
        if world == 1:
            out["cpu_baseline"] = cpu_baseline(w, fwd_only)
        print(json.dumps(out), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def reference_attention():
    """``pytorch_hstu_mha`` of the unmodified reference when its file has been placed under
    ``oracle/_ref`` (``python oracle/make_ref.py``, done by ``__graft_entry__.build()`` wherever a
    checkout of the reference is present), else None.  The two fbgemm data-movement ops it calls come
    from ``oracle/reference_shims.py``."""
    import importlib.util

    path = os.path.join(ROOT, "oracle", "_ref", "pt_hstu_attention.py")
    if not os.path.exists(path):
        return None
    try:
        from oracle import reference_shims

        reference_shims.install()
        spec = importlib.util.spec_from_file_location("_ref_pt_hstu_attention", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod.pytorch_hstu_mha
    except Exception as ex:  # pragma: no cover
        sys.stderr.write("bench: could not load oracle/_ref (%s); timing the oracle port instead\n" % ex)
        return None


def cpu_step(w, idx, fwd_only, ref_fn):
    """One pass of the CPU implementation over the sequences ``idx`` of workload ``w`` - the
    reference's own ``pytorch_hstu_mha`` when ``ref_fn`` is given, else the oracle port; returns
    (seconds, nominal forward FLOPs of those sequences)."""
    from generative_recommenders_b200 import workloads as W
    from oracle import hstu_oracle as O

    sub = W.subset(w, idx)
    q, k, v, do = sub.qkv(with_dout=True)
    q, k, v, do = (t.float() for t in (q, k, v, do))
    if not fwd_only:
        q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
    fn = ref_fn if ref_fn is not None else O.hstu_mha
    t0 = time.perf_counter()
    out = fn(sub.max_seq_len, sub.alpha, q, k, v, sub.seq_offsets, num_targets=sub.num_targets,
             max_attn_len=sub.max_attn_len, contextual_seq_len=sub.contextual_seq_len)
    if not fwd_only:
        out.backward(do)
    dt = time.perf_counter() - t0
    return dt, sub.causal_flops_fwd()


def cpu_sample(w, padded, budget=4.0e7):
    """The bounded sample the CPU legs run: the first sequences of the workload.  The oracle port
    walks the sequences (work ~ L^2 / 2 pairs per sequence and head): as many as keep the pair count
    within ``budget`` - all 64 sequences of configs[1], a handful of configs[3].  The reference
    pads every sequence to max_seq_len (work and memory ~ H * N^2 per sequence whatever its length):
    as many as keep one [n, H, N, N] fp32 tensor within ``budget`` elements, at least one."""
    if padded:
        n = int(budget // (w.num_heads * float(w.max_seq_len) ** 2))
        return list(range(max(1, min(n, len(w.lengths)))))
    idx, pairs = [], 0.0
    for i, L in enumerate(w.lengths.tolist()):
        L = min(int(L), w.max_seq_len)
        if idx and pairs + 0.5 * L * L > budget:
            break
        idx.append(i)
        pairs += 0.5 * L * L
    return idx


def _use_all_host_threads():
    # torchrun pins OMP_NUM_THREADS=1; the CPU legs may use every host core this process may run on
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except Exception:
        torch.set_num_threads(max(1, os.cpu_count() or 1))


def cpu_baseline(w, fwd_only, seconds=8.0, max_passes=200):
    """The reference's CPU implementation of the path on the host cores (the unmodified
    ``pytorch_hstu_mha`` when ``oracle/_ref`` is there, else the oracle port): passes over the
    bounded sample until ``seconds`` of CPU work have been timed."""
    _use_all_host_threads()
    ref_fn = reference_attention()
    idx = cpu_sample(w, ref_fn is not None)
    cpu_step(w, idx[:1], fwd_only, ref_fn)  # warm-up
    tot_t = tot_f = 0.0
    passes = 0
    while passes < max_passes and tot_t < seconds:
        dt, f = cpu_step(w, idx, fwd_only, ref_fn)
        tot_t += dt
        tot_f += f
        passes += 1
    mult = 1.0 if fwd_only else 3.5
    return {"value": round(mult * tot_f / tot_t / 1e12, 5), "unit": "TFLOP/s", "cores": torch.get_num_threads(),
            "kind": "reference" if ref_fn is not None else "port",
            "sample": "first %d sequences of the workload, fp32, %s, %d passes, %.1f s" % (
                len(idx), "unmodified pytorch_hstu_mha (pads to [n, H, N, N])" if ref_fn is not None
                else "oracle port (walks the sequences: faster than the reference's padded form)", passes, tot_t)}


def run_reference(args):
    """The reference's own CPU implementation of the path with all host threads: the unmodified
    ``pytorch_hstu_mha`` when ``oracle/_ref`` holds its file, else its restatement in ``oracle/``.
    The same sequences and the same number of steps whatever the number of GPUs asked for (rank 0
    alone runs; the other ranks leave at once)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    _use_all_host_threads()
    w = make_workload(1, args.workload)
    fwd_only = args.workload == "config3" or args.fwd_only
    ref_fn = reference_attention()
    idx = cpu_sample(w, ref_fn is not None)
    n = len(idx)
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_step(w, idx[:1], fwd_only, ref_fn)
    steps = max(1, min(args.steps, 100))
    tot_t = tot_f = 0.0
    done = 0
    for _ in range(steps):
        dt, f = cpu_step(w, idx, fwd_only, ref_fn)
        tot_t += dt
        tot_f += f
        done += 1
        if tot_t > 60.0:   # the whole run stays within a few minutes
            break
    steps = done
    mult = 1.0 if fwd_only else 3.5
    val = mult * tot_f / tot_t / 1e12
    kind = "reference" if ref_fn is not None else "port"
    what = "unmodified pytorch_hstu_mha" if ref_fn is not None else "oracle port"
    line = {
        "impl": "reference", "metric": "hstu_mha_%s_tflops" % ("fwd" if fwd_only else "fwd_bwd"),
        "value": round(val, 5), "unit": "TFLOP/s", "n_gpus": world, "steps": steps, "warmup": max(1, min(args.warmup, 2)),
        "ms_per_step": round(tot_t / steps * 1e3, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "configs[%s]: hstu_mha, CPU PyTorch path (%s), first %d sequences per step" % (
            "3" if fwd_only else "1", what, n)},
        "cpu_baseline": {"value": round(val, 5), "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": kind,
                         "sample": "first %d sequences per step" % n},
        "e2e": {"value": round(val, 5), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


_DIST = {}


def _dist_setup():
    """(world, rank, local_rank, device, torch.distributed or None); initialises NCCL once."""
    if _DIST:
        return _DIST["v"]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    _DIST["v"] = (world, rank, local_rank, dev, dist)
    return _DIST["v"]


def _median_ms(fn, steps, warm=2):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for s_, e_ in ev:
        s_.record()
        fn()
        e_.record()
    torch.cuda.synchronize()
    return sorted(s_.elapsed_time(e_) for s_, e_ in ev)[steps // 2]


def block_config3(dev, peaks, args):
    """configs[3] on one GPU: the inference forward in bf16 and with e4m3 q / k / v on the same
    tensors (151 MB per bf16 tensor: larger than L2), TFLOP/s over the visible (q, k) pairs."""
    import generative_recommenders_b200 as G
    from generative_recommenders_b200 import _cabi, workloads as W

    w = W.config3(256)
    q, k, v = w.qkv(device=dev)
    offs = w.seq_offsets.to(torch.int32).to(dev)
    nt = w.num_targets.to(torch.int32).to(dev)
    kw = dict(num_targets=nt, max_attn_len=w.max_attn_len)
    q8, qs, bo = G.quantize_e4m3_block(q, offs)
    k8, ks, _ = G.quantize_e4m3_block(k, offs)
    v8, vs, _ = G.quantize_e4m3_block(v, offs)
    exact = 4.0 * w.num_heads * w.attn_dim * w.exact_pairs()
    res = {"workload": "configs[3]: inference forward, B=256, N=8192, H=4, d=128, window 1024, 256 targets",
           "tokens": w.total_tokens, "flops_model": "4*H*d*(visible (q,k) pairs)"}
    with torch.no_grad():
        _cabi.profile_enable(True)
        ms16 = _median_ms(lambda: G.hstu_mha(w.max_seq_len, w.alpha, q, k, v, offs, **kw), 15)
        ms8 = _median_ms(lambda: G.hstu_mha_fp8(w.max_seq_len, w.alpha, q8, k8, v8, qs, ks, vs, bo, offs, **kw), 15)
        k16, k8_ = _cabi.profile_collect("attn_fwd"), _cabi.profile_collect("attn_fwd_fp8")
        _cabi.profile_enable(False)
        o16 = G.hstu_mha(w.max_seq_len, w.alpha, q, k, v, offs, **kw)
        o8 = G.hstu_mha_fp8(w.max_seq_len, w.alpha, q8, k8, v8, qs, ks, vs, bo, offs, **kw)
        err = float((o8.float() - o16.float()).norm() / o16.float().norm())
    for name, ms, kk, peak in (("bf16", ms16, k16, peaks["bf16_tflops"]), ("fp8", ms8, k8_, 2.0 * peaks["bf16_tflops"])):
        kms = sorted(kk)[len(kk) // 2] if kk else ms
        tf = exact / (kms * 1e-3) / 1e12
        res[name] = {"ms": round(ms, 4), "kernel_ms": round(kms, 4), "tflops_exact_pairs": round(tf, 1),
                     "frac": round(tf / peak, 4), "tokens_per_s": round(w.total_tokens / (ms * 1e-3), 1)}
    res["bf16"]["peak"] = "measured cuBLAS bf16 burst"
    res["fp8"]["peak"] = "2 x the measured bf16 burst (no fp8 GEMM was measured on this pool)"
    res["fp8"]["rel_l2_vs_bf16_kernel"] = round(err, 5)
    return res


def block_reference_gpu(dev, w, args):
    """The reference's own GPU paths on the same batch, same GPU, same run (files placed under
    ``oracle/_ref`` by ``oracle/make_ref.py``; nothing of this library is on their path): its PyTorch
    implementation (``pytorch_hstu_mha``, which pads to ``[B, H, N, N]``) forward and forward +
    backward, and the forward of its Triton kernel (``triton_hstu_mha``, autotuned by Triton itself).
    The Triton backward is left out: its sequence-parallel configurations wait on a lock in device
    memory without a bound (ops/triton/triton_attention_utils.py:42-48)."""
    ref_root = os.path.join(ROOT, "oracle", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "generative_recommenders")):
        return {"unavailable": "oracle/_ref holds no copy of the reference (python oracle/make_ref.py --reference ...)"}
    res = {"workload": "the run's configs[1] batch, bf16"}
    q, k, v, do = (t.to(dev) for t in w.qkv(with_dout=True))
    offs = w.seq_offsets.to(dev)
    nt = None if w.num_targets is None else w.num_targets.to(dev)
    flops = w.causal_flops_fwd()
    try:
        from oracle import reference_shims

        reference_shims.install()
        if ref_root not in sys.path:
            sys.path.insert(0, ref_root)
        from generative_recommenders.ops.pytorch.pt_hstu_attention import pytorch_hstu_mha

        def pt_fwd():
            with torch.no_grad():
                return pytorch_hstu_mha(w.max_seq_len, w.alpha, q, k, v, offs, num_targets=nt,
                                        max_attn_len=w.max_attn_len, contextual_seq_len=w.contextual_seq_len)

        def pt_step():
            qd, kd, vd = (t.detach().requires_grad_(True) for t in (q, k, v))
            out = pytorch_hstu_mha(w.max_seq_len, w.alpha, qd, kd, vd, offs, num_targets=nt,
                                   max_attn_len=w.max_attn_len, contextual_seq_len=w.contextual_seq_len)
            out.backward(do)

        ms_f, ms_s = _median_ms(pt_fwd, 5), _median_ms(pt_step, 5)
        res["pytorch_gpu"] = {"fwd_ms": round(ms_f, 4), "fwd_bwd_ms": round(ms_s, 4),
                              "fwd_tflops": round(flops / (ms_f * 1e-3) / 1e12, 2),
                              "fwd_bwd_tflops": round(3.5 * flops / (ms_s * 1e-3) / 1e12, 2)}
    except Exception as ex:  # pragma: no cover
        res["pytorch_gpu"] = {"unavailable": "%s: %s" % (type(ex).__name__, str(ex)[:200])}
    torch.cuda.empty_cache()
    if os.environ.get("B200_HSTU_SKIP_REFERENCE_TRITON"):
        res["triton_fwd"] = {"unavailable": "skipped on request (B200_HSTU_SKIP_REFERENCE_TRITON)"}
        return res
    try:
        from generative_recommenders.ops.triton.triton_hstu_attention import triton_hstu_mha

        def tr_fwd():
            with torch.no_grad():
                return triton_hstu_mha(w.max_seq_len, w.alpha, q, k, v, offs, num_targets=nt, max_attn_len=w.max_attn_len,
                                       contextual_seq_len=w.contextual_seq_len, sort_by_length=True)

        t0 = time.perf_counter()
        out = tr_fwd()            # autotuning happens here
        torch.cuda.synchronize()
        tune_s = time.perf_counter() - t0
        ms = _median_ms(tr_fwd, 20)
        import generative_recommenders_b200 as G

        with torch.no_grad():
            ours = G.hstu_mha(w.max_seq_len, w.alpha, q, k, v, offs, num_targets=nt, max_attn_len=w.max_attn_len,
                              contextual_seq_len=w.contextual_seq_len)
        err = float((out.float() - ours.float()).norm() / ours.float().norm())
        res["triton_fwd"] = {"ms": round(ms, 4), "tflops": round(flops / (ms * 1e-3) / 1e12, 2),
                             "autotune_s": round(tune_s, 1), "rel_l2_vs_this_library": round(err, 5)}
    except Exception as ex:  # pragma: no cover
        res["triton_fwd"] = {"unavailable": "%s: %s" % (type(ex).__name__, str(ex)[:200])}
    return res


def block_stages(dev, peaks, args):
    """Achieved HBM GB/s of the memory-bound stage kernels and TFLOP/s of the fused uvqk stage."""
    res = stage_kernels(dev, peaks, 10)
    out = {"workload": res.pop("_workload"), "hbm_peak_gb_per_s": peaks["hbm_gbs"]}
    for name, r in res.items():
        if name == "uvqk_stage":
            out[name] = {"fused_ms": r["fused"]["ms"], "separate_ms": r["separate"]["ms"],
                         "kernel_tflops": r["fused"]["kernel_tflops"],
                         "frac_of_bf16_peak": r["fused"]["kernel_frac_of_bf16_peak"], "shape": r["shape"]}
        else:
            out[name] = {"gb_per_s": r["gb_per_s"], "frac": r["frac_of_hbm_peak"], "ms": r["ms"]}
    return out


def block_config4(world, rank, dev, dist, args):
    """configs[4]: the fixed batch of 2048 sequences through the 4-layer stack (D = 1024, H = 8,
    d = 128, inference forward), split over the ranks at sequence granularity - once by token count
    (the split the configuration names) and once by estimated cost (linear stages + attention) -
    with no collective on the data path: strong scaling, tokens/s = all tokens / slowest rank."""
    import generative_recommenders_b200 as G
    from generative_recommenders_b200 import sharding, workloads as W

    w_all = W.config4(args.batch or 2048)
    D, layers, H, d = 1024, 4, 8, 128
    cfg = G.STULayerConfig(embedding_dim=D, num_heads=H, hidden_dim=d, attention_dim=d, output_dropout_ratio=0.0,
                           contextual_seq_len=16)
    torch.manual_seed(20264)
    stack = G.STUStack([G.STULayer(cfg) for _ in range(layers)]).to(dev).to(torch.bfloat16)
    stack.train(False)
    # cost of a sequence of length L in units of one token of the linear stages; the attention runs
    # at about half the GEMMs' efficiency
    per_token = 2.0 * D * 4 * H * d + 2.0 * 3 * H * d * D
    cq = 2.0 * (4.0 * H * d / 2.0) / per_token
    splits = [("by_tokens", 0.0)] + ([("by_cost", cq)] if world > 1 else [])
    res = {"workload": "configs[4]: 4-layer HSTU stack inference forward, D=1024, H=8, d=128, B=%d, N=16384, "
                       "64 targets, contextual 16, bf16" % len(w_all.lengths),
           "tokens": w_all.total_tokens, "scaling": "strong", "parallelism": "sequence-sharded x%d, no collective" % world}
    for name, c in splits:
        bins = sharding.partition_by_tokens(w_all.lengths.tolist(), world, c)
        w = W.subset(w_all, bins[rank]) if world > 1 else w_all
        g = torch.Generator(device=dev).manual_seed(w_all.seed + 7 + rank)
        x = torch.randn(w.total_tokens, D, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
        lengths = w.lengths.to(dev)
        offs = w.seq_offsets.to(torch.int32).to(dev)
        nt = w.num_targets.to(torch.int32).to(dev)
        with torch.no_grad():
            fn = lambda: stack(x, lengths, offs, w.max_seq_len, nt)  # noqa: E731
            fn()
            torch.cuda.synchronize()
            if dist is not None:
                dist.barrier()
            ms = _median_ms(fn, 3, warm=0)
        lsq = float((w.lengths.double() ** 2).sum())
        mine = torch.tensor([ms, float(w.total_tokens), lsq], dtype=torch.float64, device=dev)
        if dist is not None:
            allr = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(allr, mine)
            allr = torch.stack(allr).cpu()
        else:
            allr = mine.cpu().view(1, -1)
        slow = float(allr[:, 0].max())
        res[name] = {"tokens_per_s": round(w_all.total_tokens / (slow * 1e-3), 1), "ms": round(slow, 3),
                     "rank_ms": {"min": round(float(allr[:, 0].min()), 3), "max": round(slow, 3),
                                 "argmax": int(allr[:, 0].argmax())},
                     "rank_tokens": {"min": int(allr[:, 1].min()), "max": int(allr[:, 1].max())},
                     "rank_sum_L2": {"min": float(allr[:, 2].min()), "max": float(allr[:, 2].max())}}
        del x
        torch.cuda.empty_cache()
    best = max((k_ for k_ in ("by_tokens", "by_cost") if k_ in res), key=lambda k_: res[k_]["tokens_per_s"])
    res["tokens_per_s"] = res[best]["tokens_per_s"]
    res["best_split"] = best
    return res


def run_stack(args):
    """configs[2]: 8-layer HSTU stack, D=512, H=4, d=128, forward + backward (training step without the
    optimizer: the path is the layer stack), bf16, relative bias on.  configs[4]: 4-layer stack, D=1024,
    H=8, d=128, inference forward; the fixed batch is split over the ranks by token count (strong
    scaling), no collective on the data path."""
    import generative_recommenders_b200 as G
    from generative_recommenders_b200 import _cabi, sharding, workloads as W

    world, rank, local_rank, dev, dist = _dist_setup()
    train = args.workload == "config2_stack"
    if train:
        w_all = W.config2_attention(args.batch or 128)
        # 8 505 tokens: activations are kept (the recompute switches, which trade memory for one more
        # launch of two kernels per layer in the backward, are off); the bias tables are trained
        D, layers, cfg = 512, 8, G.STULayerConfig(embedding_dim=512, num_heads=4, hidden_dim=128, attention_dim=128,
                                                  output_dropout_ratio=0.0, contextual_seq_len=6, rel_bias_buckets=128,
                                                  recompute_normed_x=False, recompute_uvqk=False, recompute_y=False)
    else:
        w_all = W.config4(args.batch or 2048)
        D, layers, cfg = 1024, 4, G.STULayerConfig(embedding_dim=1024, num_heads=8, hidden_dim=128, attention_dim=128,
                                                   output_dropout_ratio=0.0, contextual_seq_len=16)
    bins = sharding.partition_by_tokens(w_all.lengths.tolist(), world)
    w = W.subset(w_all, bins[rank]) if world > 1 else w_all
    torch.manual_seed(20260 + (2 if train else 4))
    stack = G.STUStack([G.STULayer(cfg) for _ in range(layers)]).to(dev).to(torch.bfloat16)
    stack.train(False)
    g = torch.Generator().manual_seed(w_all.seed + 7 + rank)
    L = w.total_tokens
    hx = torch.randn(L, D, generator=g).to(torch.bfloat16).pin_memory()
    hdy = torch.randn(L, D, generator=g).to(torch.bfloat16).pin_memory() if train else None
    x = hx.to(dev)
    dy = hdy.to(dev) if train else None
    lengths = w.lengths.to(dev)
    offs = w.seq_offsets.to(torch.int32).to(dev)
    nt = w.num_targets.to(torch.int32).to(dev)
    N = w.max_seq_len
    params = [p_ for p_ in stack.parameters()]

    def step(xin, dyin):
        if train:
            xin = xin.detach().requires_grad_(True)
            for p_ in params:
                p_.grad = None
            y = stack(xin, lengths, offs, N, nt)
            y.backward(dyin)
            return y, xin.grad
        with torch.no_grad():
            return stack(xin, lengths, offs, N, nt), None

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step(x, dy)
    barrier()
    graph = None
    if args.graph and train:
        sx, sdy = x.clone(), dy.clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                step(sx, sdy)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            gy, gdx = step(sx, sdy)
        run = graph.replay
    else:
        run = lambda: step(x, dy)  # noqa: E731
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    steps = args.steps
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    launches0 = _cabi.launch_count()
    with ClockSampler(local_rank) as clocks:
        barrier()
        for s_, e_ in ev:
            flush.zero_()
            s_.record()
            run()
            e_.record()
        barrier()
    launches = _cabi.launch_count() - launches0
    ms_total = sum(s_.elapsed_time(e_) for s_, e_ in ev)
    # end to end: pinned host activations in, result back
    res_host = torch.empty_like(hx)
    e2e_steps = max(2, min(steps, 5))

    def e2e_step():
        xd = hx.to(dev, non_blocking=True)
        dyd = hdy.to(dev, non_blocking=True) if train else None
        y, dx = step(xd, dyd)
        res_host.copy_(dx if train else y, non_blocking=True)

    e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    stats = torch.tensor([ms_total, e2e_ms], dtype=torch.float64, device=dev)
    work = torch.tensor([float(L), w.causal_flops_fwd() * layers, float(launches)], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(work, op=dist.ReduceOp.SUM)
    ms_total, e2e_ms = stats.tolist()
    tokens_all, attn_flops_all, launches_all = work.tolist()
    ms_per_step = ms_total / steps
    if rank == 0:
        H, d = cfg.num_heads, cfg.attention_dim
        gemm_flops = tokens_all * layers * (2.0 * D * 4 * H * d + 2.0 * 3 * H * d * D)
        mult = 3.0 if train else 1.0
        out = {
            "metric": "hstu_stack_tokens_per_s", "value": round(tokens_all / (ms_per_step * 1e-3), 1), "unit": "tokens/s",
            "n_gpus": world, "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": True, "scaling": "strong" if not train else "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": "configs[%s]: %d-layer HSTU stack %s, D=%d, H=%d, d=%d, B=%d, N=%d%s" % (
                "2" if train else "4", layers, "fwd+bwd" if train else "inference fwd", D, H, d, len(w_all.lengths), N,
                ", CUDA graph replay" if graph is not None else ""),
                "global_batch": len(w_all.lengths), "tokens": int(tokens_all), "seq_len": N,
                "parallelism": "sequence-sharded x%d by token count, no collective" % world,
                "l2": "256 MiB memset between timed steps (untimed)"},
            "attn_tflops_nominal": round((3.5 if train else 1.0) * attn_flops_all / (ms_per_step * 1e-3) / 1e12, 2),
            "total_tflops_nominal": round((mult * gemm_flops + (3.5 if train else 1.0) * attn_flops_all) /
                                          (ms_per_step * 1e-3) / 1e12, 2),
            "e2e": {"value": round(tokens_all / (e2e_ms * 1e-3), 1), "unit": "tokens/s",
                    "h2d_bytes_per_step": int(hx.numel() * 2 * (2 if train else 1)), "d2h_bytes_per_step": int(hx.numel() * 2),
                    "ms_per_step": round(e2e_ms, 4)},
            "gpu_launches": int(launches_all), "clocks": clocks.summary(),
        }
        print(json.dumps(out), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_fp8(args):
    """configs[3] inference forward with e4m3 q/k/v (per-128-token-block scales) next to the bf16 run of the
    same tensors."""
    import generative_recommenders_b200 as G
    from generative_recommenders_b200 import _cabi, workloads as W
    from oracle import hstu_oracle as O

    world, rank, local_rank, dev, dist = _dist_setup()
    w = W.config3(args.batch or 256)
    q, k, v = w.qkv(device=dev)
    offs = w.seq_offsets.to(torch.int32).to(dev)
    nt = w.num_targets.to(torch.int32).to(dev)
    q8, qs, bo = G.quantize_e4m3_block(q, offs)
    k8, ks, _ = G.quantize_e4m3_block(k, offs)
    v8, vs, _ = G.quantize_e4m3_block(v, offs)
    kw = dict(num_targets=nt, max_attn_len=w.max_attn_len)
    f8 = lambda: G.hstu_mha_fp8(w.max_seq_len, w.alpha, q8, k8, v8, qs, ks, vs, bo, offs, **kw)  # noqa: E731
    f16 = lambda: G.hstu_mha(w.max_seq_len, w.alpha, q, k, v, offs, **kw)  # noqa: E731
    with torch.no_grad():
        for _ in range(max(args.warmup, 3)):
            o8 = f8()
            o16 = f16()
        torch.cuda.synchronize()
        err = O.rel_l2(o8, o16)
        res = {}
        _cabi.profile_enable(True)
        for name, fn in (("fp8", f8), ("bf16", f16)):
            ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
            for s_, e_ in ev:
                s_.record()
                fn()
                e_.record()
            torch.cuda.synchronize()
            res[name] = sum(s_.elapsed_time(e_) for s_, e_ in ev) / args.steps
        kms = {kk: (lambda vv: sum(vv) / len(vv) if vv else None)(_cabi.profile_collect(kk)) for kk in ("attn_fwd_fp8", "attn_fwd")}
        _cabi.profile_enable(False)
    exact = 4.0 * w.num_heads * w.attn_dim * w.exact_pairs()
    out = {
        "metric": "hstu_mha_fwd_fp8_tflops_exact_pairs", "value": round(exact / (res["fp8"] * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(res["fp8"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "e4m3 (fp32 accumulate, bf16 out)",
        "data": "synthetic",
        "config": {"workload": "configs[3]: inference forward, B=%d, N=8192, H=4, d=128, window 1024, 256 targets; "
                               "inputs (%.0f MB per tensor in bf16) are larger than L2" % (len(w.lengths), q.numel() * 2 / 1e6),
                   "tokens": w.total_tokens},
        "bf16_ms": round(res["bf16"], 4), "bf16_tflops_exact_pairs": round(exact / (res["bf16"] * 1e-3) / 1e12, 2),
        "nominal_causal_tflops_fp8": round(w.causal_flops_fwd() / (res["fp8"] * 1e-3) / 1e12, 2),
        "kernel_ms": kms, "rel_l2_fp8_vs_bf16": round(err, 5), "tokens_per_s": round(w.total_tokens / (res["fp8"] * 1e-3), 1),
    }
    print(json.dumps(out), flush=True)


def _uvqk_stage(dev, peaks, steps):
    """The uvqk stage at configs[1]'s token count (D = 512, H = 4, d = 128): one fused tensor-core
    kernel against LayerNorm kernel + library GEMM + SiLU kernel, forward only."""
    import generative_recommenders_b200 as G
    from generative_recommenders_b200 import _cabi, hstu_compute as HC, workloads as W

    D, H_, d_ = 512, 4, 128
    g = torch.Generator().manual_seed(5)
    mk = lambda *shape: torch.randn(*shape, generator=g).to(torch.bfloat16).to(dev)  # noqa: E731
    uq_rows = int(W.config1().total_tokens)
    xs, w_, b_ = mk(uq_rows, D), mk(D), mk(D)
    Wu = (torch.randn(D, 4 * H_ * d_, generator=g) / D ** 0.5).to(torch.bfloat16).to(dev)
    bu = mk(4 * H_ * d_)
    uq = {}
    for name, fused in (("fused", True), ("separate", False)):
        HC.set_fused_uqvk(fused)
        with torch.no_grad():
            fn = lambda: G.hstu_compute_uqvk(xs, w_, b_, 1e-6, H_, d_, d_, Wu, bu)  # noqa: E731
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
            for s_, e_ in ev:
                s_.record()
                fn()
                e_.record()
            torch.cuda.synchronize()
        ms = sorted(s_.elapsed_time(e_) for s_, e_ in ev)[steps // 2]
        uq[name] = {"ms": round(ms, 4), "tflops": round(2.0 * uq_rows * D * Wu.shape[1] / (ms * 1e-3) / 1e12, 1)}
    HC.set_fused_uqvk(True)
    _cabi.profile_enable(True)
    with torch.no_grad():
        for _ in range(max(steps, 3)):
            G.hstu_compute_uqvk(xs, w_, b_, 1e-6, H_, d_, d_, Wu, bu)
    torch.cuda.synchronize()
    kk = _cabi.profile_collect("ln_linear")
    kp = _cabi.profile_collect("ln_linear_prep")
    _cabi.profile_enable(False)
    kms = sorted(kk)[len(kk) // 2]
    uq["fused"]["kernel_ms"] = round(kms, 4)
    uq["fused"]["prep_ms"] = round(sorted(kp)[len(kp) // 2], 4)
    uq["fused"]["kernel_tflops"] = round(2.0 * uq_rows * D * Wu.shape[1] / (kms * 1e-3) / 1e12, 1)
    uq["fused"]["kernel_frac_of_bf16_peak"] = round(uq["fused"]["kernel_tflops"] / peaks["bf16_tflops"], 3)
    uq["rows"] = uq_rows
    uq["shape"] = "x [%d, %d] -> uvqk [%d, %d], u [%d, %d]" % (uq_rows, D, uq_rows, Wu.shape[1], uq_rows, H_ * d_)
    return uq


def run_uvqk(args):
    """``--workload uvqk``: the fused uvqk stage alone (a small case for profiling)."""
    world, rank, local_rank, dev, dist = _dist_setup()
    peaks, peak_kind = load_peaks()
    uq = _uvqk_stage(dev, peaks, max(3, min(args.steps, 30)))
    out = {"metric": "hstu_uvqk_stage_tflops", "value": uq["fused"]["tflops"], "unit": "TFLOP/s", "n_gpus": 1,
           "steps": args.steps, "warmup": 3, "ms_per_step": uq["fused"]["ms"], "higher_is_better": True,
           "dtype": "bf16", "data": "synthetic", "config": {"workload": "uvqk stage forward, " + uq["shape"]},
           "bf16_peak_tflops": peaks["bf16_tflops"], "peak_source": peak_kind + " (cuBLAS bf16 burst)", "uvqk_stage": uq}
    print(json.dumps(out), flush=True)


def run_norm_mul(args):
    """``--workload norm_mul``: the output stage's norm-mul kernel alone on [131 072, 512] bf16 with the
    ``[u | attn | y]`` concatenation (the two inputs 134 MB each, the output and its gradient 403 MB each,
    about 1.5 GB on the device - a case sized for profiling): forward and backward without dropout, with
    dropout, and the backward once from the forward's stored mask bits and once regenerating the mask."""
    import generative_recommenders_b200 as G
    from generative_recommenders_b200 import _cabi

    world, rank, local_rank, dev, dist = _dist_setup()
    peaks, peak_kind = load_peaks()
    rows, H, V = 131072, 4, 128
    D = H * V
    g = torch.Generator().manual_seed(5)
    mk = lambda *shape: torch.randn(*shape, generator=g).to(torch.bfloat16).to(dev)  # noqa: E731
    attn, u, w_, b_, dcat = mk(rows, D), mk(rows, D), mk(D), mk(D), mk(rows, 3 * D)
    ar, ur, wr, br = (t.clone().requires_grad_(True) for t in (attn, u, w_, b_))
    seed = torch.tensor([20260], dtype=torch.int64, device=dev)
    fwd = lambda p, *t: G.hstu_norm_mul_dropout(*t, 1e-6, p, p > 0, True, True, "none", False, H, V,  # noqa: E731
                                                dropout_seed=seed if p > 0 else None)
    y_plain = fwd(0.0, ar, ur, wr, br)
    y_regen = fwd(0.3, ar, ur, wr, br)
    G.hstu_compute.set_store_dropout_mask(True)
    y_bits = fwd(0.3, ar, ur, wr, br)
    G.hstu_compute.set_store_dropout_mask(False)
    bwd = lambda y: torch.autograd.grad(y, (ar, ur, wr, br), dcat, retain_graph=True)  # noqa: E731

    def fwd_bits():
        G.hstu_compute.set_store_dropout_mask(True)
        try:
            return fwd(0.3, ar, ur, wr, br)
        finally:
            G.hstu_compute.set_store_dropout_mask(False)

    fb, bb = rows * D * 2 * 5 + rows * 8, rows * D * 2 * 7 + rows * 8
    steps = max(3, min(args.steps, 30))
    res = {}
    for name, kind, fn, nbytes in (("fwd", "norm_mul_fwd", lambda: fwd(0.0, attn, u, w_, b_), fb),
                                   ("bwd", "norm_mul_bwd", lambda: bwd(y_plain), bb),
                                   ("fwd_dropout", "norm_mul_fwd", lambda: fwd(0.3, attn, u, w_, b_), fb),
                                   ("fwd_dropout_keeping_bits", "norm_mul_fwd", lambda: fwd_bits(), fb + rows * 3 * D // 8),
                                   ("bwd_dropout_stored_bits", "norm_mul_bwd", lambda: bwd(y_bits), bb + rows * 3 * D // 8),
                                   ("bwd_dropout_regenerated", "norm_mul_bwd", lambda: bwd(y_regen), bb)):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        _cabi.profile_enable(True)
        for _ in range(steps):
            fn()
        torch.cuda.synchronize()
        v = _cabi.profile_collect(kind)
        _cabi.profile_enable(False)
        ms = sorted(v)[len(v) // 2]
        gbs = nbytes / (ms * 1e-3) / 1e9
        res[name] = {"ms": round(ms, 4), "bytes": int(nbytes), "gb_per_s": round(gbs, 1),
                     "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 3)}
    out = {"metric": "norm_mul_hbm_gb_per_s", "value": res["fwd"]["gb_per_s"], "unit": "GB/s", "n_gpus": 1,
           "steps": steps, "warmup": 3, "ms_per_step": res["fwd"]["ms"], "higher_is_better": True,
           "dtype": "bf16", "data": "synthetic",
           "config": {"workload": "norm-mul forward / backward, rows=%d, D=%d, [u | attn | y] output" % (rows, D)},
           "hbm_peak_gb_per_s": peaks["hbm_gbs"], "peak_source": peak_kind + " (copy)", "stages": res}
    print(json.dumps(out), flush=True)


def run_layer_norm(args):
    """``--workload layer_norm``: LayerNorm forward / backward alone on [655 360, 512] bf16 (671 MB per
    tensor, larger than L2; about 3 GB on the device - a case sized for profiling)."""
    import generative_recommenders_b200 as G
    from generative_recommenders_b200 import _cabi

    world, rank, local_rank, dev, dist = _dist_setup()
    peaks, peak_kind = load_peaks()
    rows, D = 655360, 512
    g = torch.Generator().manual_seed(5)
    x = torch.randn(rows, D, generator=g).to(torch.bfloat16).to(dev)
    dy = torch.randn(rows, D, generator=g).to(torch.bfloat16).to(dev)
    w_ = torch.randn(D, generator=g).to(torch.bfloat16).to(dev)
    b_ = torch.randn(D, generator=g).to(torch.bfloat16).to(dev)
    xr, wr, br = (t.clone().requires_grad_(True) for t in (x, w_, b_))
    y = G.layer_norm(xr, wr, br, 1e-6)
    steps = max(3, min(args.steps, 30))
    res = {}
    for kind, fn, nbytes in (("layer_norm_fwd", lambda: G.layer_norm(x, w_, b_, 1e-6), rows * D * 2 * 2 + rows * 8),
                             ("layer_norm_bwd", lambda: torch.autograd.grad(y, (xr, wr, br), dy, retain_graph=True),
                              rows * D * 2 * 3 + rows * 8)):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        _cabi.profile_enable(True)
        for _ in range(steps):
            fn()
        torch.cuda.synchronize()
        v = _cabi.profile_collect(kind)
        _cabi.profile_enable(False)
        ms = sorted(v)[len(v) // 2]
        gbs = nbytes / (ms * 1e-3) / 1e9
        res[kind] = {"ms": round(ms, 4), "bytes": int(nbytes), "gb_per_s": round(gbs, 1),
                     "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 3)}
    out = {"metric": "layer_norm_hbm_gb_per_s", "value": res["layer_norm_fwd"]["gb_per_s"], "unit": "GB/s", "n_gpus": 1,
           "steps": steps, "warmup": 3, "ms_per_step": res["layer_norm_fwd"]["ms"], "higher_is_better": True,
           "dtype": "bf16", "data": "synthetic",
           "config": {"workload": "LayerNorm forward / backward, rows=%d, D=%d (tensors of %.0f MB, larger than L2)"
                                  % (rows, D, rows * D * 2 / 1e6)},
           "hbm_peak_gb_per_s": peaks["hbm_gbs"], "peak_source": peak_kind + " (copy)", "stages": res}
    print(json.dumps(out), flush=True)


def stage_kernels(dev, peaks, steps):
    """Achieved HBM GB/s of the memory-bound stage kernels (bf16, D = H*dv = 512, rows = tokens of
    configs[4]'s first 400 sequences), from the library's per-kernel events."""
    import generative_recommenders_b200 as G
    from generative_recommenders_b200 import _cabi, workloads as W

    rows = int(W.config4(400).total_tokens)
    D = 512
    g = torch.Generator().manual_seed(5)
    mk = lambda *shape: torch.randn(*shape, generator=g).to(torch.bfloat16).to(dev)  # noqa: E731
    x, dy = mk(rows, D), mk(rows, D)
    w_, b_ = mk(D), mk(D)
    uvqk = mk(rows, 4 * D)
    attn, u, dcat = mk(rows, D), mk(rows, D), mk(rows, 3 * D)

    def timed(kind, fn, nbytes):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        _cabi.profile_enable(True)
        for _ in range(max(5, min(steps, 30))):
            fn()
        torch.cuda.synchronize()
        v = _cabi.profile_collect(kind)
        _cabi.profile_enable(False)
        ms = sorted(v)[len(v) // 2]
        gbs = nbytes / (ms * 1e-3) / 1e9
        return {"ms": round(ms, 4), "bytes": int(nbytes), "gb_per_s": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 3)}

    res = {}
    xr = x.clone().requires_grad_(True)
    wr = w_.clone().requires_grad_(True)
    br = b_.clone().requires_grad_(True)
    res["layer_norm_fwd"] = timed("layer_norm_fwd", lambda: G.layer_norm(x, w_, b_, 1e-6), rows * D * 2 * 2 + rows * 8)
    y = G.layer_norm(xr, wr, br, 1e-6)
    res["layer_norm_bwd"] = timed("layer_norm_bwd", lambda: torch.autograd.grad(y, (xr, wr, br), dy, retain_graph=True),
                                  rows * D * 2 * 3 + rows * 8)
    res["silu_u"] = timed("silu", lambda: G.hstu_compute._SiluColumnsFunction.apply(uvqk[:, :D], D), rows * D * 2 * 2)
    res["norm_mul_fwd"] = timed("norm_mul_fwd", lambda: G.hstu_norm_mul_dropout(attn, u, w_, b_, 1e-6, 0.0, False, True, True,
                                                                                  "none", False, 4, 128), rows * D * 2 * 5 + rows * 8)
    ar = attn.clone().requires_grad_(True)
    ur = u.clone().requires_grad_(True)
    yc = G.hstu_norm_mul_dropout(ar, ur, wr, br, 1e-6, 0.0, False, True, True, "none", False, 4, 128)
    res["norm_mul_bwd"] = timed("norm_mul_bwd", lambda: torch.autograd.grad(yc, (ar, ur, wr, br), dcat, retain_graph=True),
                                rows * D * 2 * 7 + rows * 8)
    # training: the dropout mask is generated inside the same kernels (same algorithmic bytes; a
    # separate dropout pass would move another 6 * D * 2 bytes per row and keep a mask)
    seed = torch.tensor([20260], dtype=torch.int64, device=dev)
    res["norm_mul_fwd_dropout"] = timed("norm_mul_fwd", lambda: G.hstu_norm_mul_dropout(
        attn, u, w_, b_, 1e-6, 0.3, True, True, True, "none", False, 4, 128, dropout_seed=seed), rows * D * 2 * 5 + rows * 8)
    # backward: regenerates the mask from the seed (the default), or - switched on - reads the bits the
    # forward kept (one bit per output element, + 3 * D / 8 bytes per row each way)
    yd = G.hstu_norm_mul_dropout(ar, ur, wr, br, 1e-6, 0.3, True, True, True, "none", False, 4, 128, dropout_seed=seed)
    res["norm_mul_bwd_dropout"] = timed("norm_mul_bwd", lambda: torch.autograd.grad(yd, (ar, ur, wr, br), dcat, retain_graph=True),
                                        rows * D * 2 * 7 + rows * 8)
    G.hstu_compute.set_store_dropout_mask(True)
    res["norm_mul_fwd_dropout_keeping_bits"] = timed("norm_mul_fwd", lambda: G.hstu_norm_mul_dropout(
        ar, ur, wr, br, 1e-6, 0.3, True, True, True, "none", False, 4, 128, dropout_seed=seed),
        rows * D * 2 * 5 + rows * 8 + rows * 3 * D // 8)
    yd = G.hstu_norm_mul_dropout(ar, ur, wr, br, 1e-6, 0.3, True, True, True, "none", False, 4, 128, dropout_seed=seed)
    G.hstu_compute.set_store_dropout_mask(False)
    res["norm_mul_bwd_dropout_stored_bits"] = timed(
        "norm_mul_bwd", lambda: torch.autograd.grad(yd, (ar, ur, wr, br), dcat, retain_graph=True),
        rows * D * 2 * 7 + rows * 8 + rows * 3 * D // 8)
    del yd
    # jagged glue: KV-cache split / concat of [rows, H*d] K rows (last 20 rows of every sequence on
    # the right), and the timestamp + position embedding step before layer 0
    from generative_recommenders_b200.jagged_tensors import concat_2D_jagged, split_2D_jagged
    from generative_recommenders_b200.position import add_timestamp_positional_embeddings
    wl = W.config4(400)
    lengths = wl.lengths.to(dev)
    offs = torch.cat([lengths.new_zeros(1), torch.cumsum(lengths, 0)])
    prime_offs = torch.cat([lengths.new_zeros(1), torch.cumsum(lengths - 20, 0)])
    n_left = rows - 20 * len(wl.lengths)
    res["split_2D_jagged"] = timed("jagged", lambda: split_2D_jagged(0, x, n_left, rows - n_left, None, 20, prime_offs, None),
                                   rows * D * 2 * 2)
    left, right = split_2D_jagged(0, x, n_left, rows - n_left, None, 20, prime_offs, None)
    res["concat_2D_jagged"] = timed("jagged", lambda: concat_2D_jagged(0, left, right, None, 20, prime_offs, None),
                                    rows * D * 2 * 2)
    pos_w = torch.randn(16384 + 1, D, device=dev) * 0.1
    ts_w = torch.randn(2048 + 1, D, device=dev) * 0.1
    gaps = (torch.rand(rows, generator=g) * 12).exp().long().to(dev)
    stamps = torch.cumsum(gaps, 0)  # increasing inside every sequence
    nt = wl.num_targets.to(dev)
    xe = x.clone().requires_grad_(True)
    pw = pos_w.clone().requires_grad_(True)
    tw = ts_w.clone().requires_grad_(True)
    emb = lambda a, p_, t_: add_timestamp_positional_embeddings(  # noqa: E731
        D ** 0.5, 16384, 0, p_, t_, offs, lengths, a, stamps, nt, False, "sqrt")
    with torch.no_grad():
        res["add_timestamp_positional_embeddings_fwd"] = timed("ts_pos", lambda: emb(x, pos_w, ts_w), rows * D * 2 * 2)
    ye = emb(xe, pw, tw)
    res["add_timestamp_positional_embeddings_bwd"] = timed(
        "ts_pos", lambda: torch.autograd.grad(ye, (xe, pw, tw), dy, retain_graph=True), rows * D * 2 * 2)
    res["uvqk_stage"] = _uvqk_stage(dev, peaks, 20)
    # the same stage kernels at configs[4]'s width (D = H * dv = 1024: four 16-byte vectors per lane), half the rows
    del ye, left, right, yc, y
    rows2, D2 = rows // 2, 1024
    x2, dy2, w2, b2 = mk(rows2, D2), mk(rows2, D2), mk(D2), mk(D2)
    u2, dcat2 = mk(rows2, D2), mk(rows2, 3 * D2)
    x2r, u2r, w2r, b2r = (t.clone().requires_grad_(True) for t in (x2, u2, w2, b2))
    res["layer_norm_fwd_d1024"] = timed("layer_norm_fwd", lambda: G.layer_norm(x2, w2, b2, 1e-6), rows2 * D2 * 2 * 2 + rows2 * 8)
    y2 = G.layer_norm(x2r, w2r, b2r, 1e-6)
    res["layer_norm_bwd_d1024"] = timed("layer_norm_bwd", lambda: torch.autograd.grad(y2, (x2r, w2r, b2r), dy2, retain_graph=True),
                                        rows2 * D2 * 2 * 3 + rows2 * 8)
    nm2 = lambda p_, *t: G.hstu_norm_mul_dropout(*t, 1e-6, p_, p_ > 0, True, True, "none", False, 8, 128,  # noqa: E731
                                                 dropout_seed=seed if p_ > 0 else None)
    res["norm_mul_fwd_d1024"] = timed("norm_mul_fwd", lambda: nm2(0.0, x2, u2, w2, b2), rows2 * D2 * 2 * 5 + rows2 * 8)
    res["norm_mul_fwd_dropout_d1024"] = timed("norm_mul_fwd", lambda: nm2(0.3, x2, u2, w2, b2), rows2 * D2 * 2 * 5 + rows2 * 8)
    for name, p_ in (("norm_mul_bwd_d1024", 0.0), ("norm_mul_bwd_dropout_d1024", 0.3)):
        yc2 = nm2(p_, x2r, u2r, w2r, b2r)
        res[name] = timed("norm_mul_bwd", lambda: torch.autograd.grad(yc2, (x2r, u2r, w2r, b2r), dcat2, retain_graph=True),
                          rows2 * D2 * 2 * 7 + rows2 * 8)
        del yc2
    res["_workload"] = ("stage kernels, rows=%d, D=H*dv=512 (tensors of %.0f MB, larger than L2); *_d1024: rows=%d, D=1024"
                        % (rows, rows * D * 2 / 1e6, rows2))
    return res


def run_stages(args):
    """``--workload stages``: the stage kernels alone."""
    world, rank, local_rank, dev, dist = _dist_setup()
    peaks, peak_kind = load_peaks()
    res = stage_kernels(dev, peaks, args.steps)
    workload = res.pop("_workload")
    out = {"metric": "hstu_stage_hbm_gb_per_s", "value": res["norm_mul_fwd"]["gb_per_s"], "unit": "GB/s", "n_gpus": 1,
           "steps": args.steps, "warmup": 3, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
           "config": {"workload": workload},
           "hbm_peak_gb_per_s": peaks["hbm_gbs"], "peak_source": peak_kind + " (copy)", "stages": res}
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="config1",
                    choices=["config1", "config3", "config3_fp8", "config2_stack", "config4_stack", "stages", "uvqk", "layer_norm", "norm_mul"])
    ap.add_argument("--graph", action="store_true", help="config2_stack: replay the step from a CUDA graph")
    ap.add_argument("--batch", type=int, default=0, help="override the number of sequences (stack workloads)")
    ap.add_argument("--fwd-only", action="store_true", help="time the forward alone (inference)")
    ap.add_argument("--eager", action="store_true", help="time eager launches instead of replaying a CUDA graph of the step")
    ap.add_argument("--rounds", type=int, default=0,
                    help="rounds of --steps timed steps (default: as many as fill half a second; profiling runs pass 1)")
    ap.add_argument("--blocks", default="all", choices=["all", "none"],
                    help="none: leave out the configs[3] / stage-kernel / configs[4] records (profiling runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload in ("config2_stack", "config4_stack"):
        run_stack(args)
    elif args.workload == "stages":
        run_stages(args)
    elif args.workload == "uvqk":
        run_uvqk(args)
    elif args.workload == "layer_norm":
        run_layer_norm(args)
    elif args.workload == "norm_mul":
        run_norm_mul(args)
    elif args.workload == "config3_fp8":
        run_fp8(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
