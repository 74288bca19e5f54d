"""Benchmark of the block-sparse attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" = one pass of the hot path over one batch of synthetic input: draw the block mask on
the device, compact it into index lists (both directions), forward, backward.  The workload is the
one the metric is quoted on: dynamic random block-sparse attention, B=1, H=24, D=128,
q_block=kv_block=384, S=69120, Bernoulli(keep 0.4) per-(batch, head) mask with the diagonal
forced on, q,k,v,dO ~ N(0,1) bf16 from a seed.  With N GPUs the 24 heads are split evenly over
the ranks (no data-path collective; strong scaling: total work is fixed).

The printed line carries
  value      whole-job effective TFLOPS (14*qb*kb*D FLOPs per active block pair, active blocks
             only), inputs resident in HBM, CUDA events, max over ranks;
  e2e        the same metric through the public API (flex_block_attn_func + backward) with q, k, v,
             dO copied from pinned host memory and a checksum read back inside the timed region;
  roofline   the backward main kernel (largest share of the step) against the measured dense
             bf16 peak, timed live with CUDA events recorded around that kernel alone;
  cpu_baseline  torch dense-masked SDPA (the reference's own oracle path) on the host cores, on a
             bounded sample of the same workload.
`--impl reference` times only that CPU path (the reference's CUDA kernels are Hopper-only and
their ThunderKittens dependency is not vendored, so they cannot run on this machine).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

QB = KB = 384
D = 128
FLOPS_PER_PAIR_FWD = 4 * QB * KB * D
FLOPS_PER_PAIR_BWD = 10 * QB * KB * D
FLOPS_PER_PAIR = FLOPS_PER_PAIR_FWD + FLOPS_PER_PAIR_BWD
METRIC = "fwd+bwd effective TFLOPS (active blocks), S=69120 sparse 0.6; % B200 bf16 peak"

# DRAM traffic of the backward main kernel per active 384x384 block pair, from the ncu capture
# summarised under profiles/ (backward kernel, S=23040 H=8 case): (dram__bytes_read.sum + dram__bytes_write.sum)
# = 431.0 MB for the 11 805 pairs of the captured launch.  The bench workload is too large to capture
# under the size rule, so `roofline.traffic` scales this figure by the pairs of a full launch; in
# the captured case the dQ accumulator is L2-resident, at full size it is not, so the true figure is
# higher than this proportional scaling.
BWD_DRAM_BYTES_PER_PAIR = 431.0e6 / 11805


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--seq", type=int, default=69120)
    ap.add_argument("--heads", type=int, default=24)
    ap.add_argument("--keep", type=float, default=0.4)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"burst": float(d["bf16_tflops"]), "sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"burst": 1590.0, "sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle-reason sampling during the timed region (read-only query)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "50"], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        try:
            for line in Path(self.path).read_text().splitlines():
                parts = [x.strip() for x in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                except ValueError:
                    continue
                try:
                    pw.append(float(parts[3]))
                except ValueError:
                    pass
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no_samples"]}
        out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}
        if pw:
            out["power_w"] = statistics.median(pw)
        return out


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except (ValueError, IndexError):
            pass
    return local_rank


# ------------------------------------------------------------------------------------------------
# CPU path (the reference's torch oracle) on a bounded sample of the workload
# ------------------------------------------------------------------------------------------------
def cpu_sample_run(S: int, keep: float, n_qblocks: int, seed: int = 1234):
    """fwd+bwd of `n_qblocks` query blocks of one head against all S keys; returns (seconds, pairs)."""
    from oracle import dense_oracle as orc

    g = torch.Generator().manual_seed(seed)
    nb = S // KB
    q = torch.randn((1, 1, n_qblocks * QB, D), generator=g).requires_grad_()
    k = torch.randn((1, 1, S, D), generator=g).requires_grad_()
    v = torch.randn((1, 1, S, D), generator=g).requires_grad_()
    do = torch.randn((1, 1, n_qblocks * QB, D), generator=g)
    mask = torch.rand((n_qblocks, nb), generator=g) < keep
    mask[torch.arange(n_qblocks), torch.arange(n_qblocks)] = True
    t0 = time.perf_counter()
    o = orc.sdpa_dense(q, k, v, mask, QB, KB)
    o.backward(do)
    dt = time.perf_counter() - t0
    return dt, int(mask.sum())


def use_all_host_threads() -> int:
    """torchrun pins OMP_NUM_THREADS=1; the CPU legs are meant to use every host core."""
    n = os.cpu_count() or 1
    try:
        n = len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        pass
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def cpu_baseline(S: int, keep: float, target_s: float = 12.0):
    threads = use_all_host_threads()
    cpu_sample_run(min(S, 3840), keep, 1)  # warm-up of the torch CPU kernels
    nq = 8 if S >= 8 * QB else max(1, S // QB)
    dt, pairs = cpu_sample_run(S, keep, nq)
    reps = max(1, min(24, int(round(target_s / max(dt, 1e-3)))))
    for r in range(1, reps):
        d, p = cpu_sample_run(S, keep, nq, seed=1234 + r)
        dt += d
        pairs += p
    tflops = pairs * FLOPS_PER_PAIR / dt / 1e12
    return {"value": tflops, "unit": "TFLOPS", "cores": threads, "kind": "port",
            "sample": f"torch F.scaled_dot_product_attention + dense token mask (the reference's oracle path), fp32, "
                      f"fwd+bwd of {reps} x {nq} query blocks of one head against all {S} keys of the S={S} keep={keep} workload, "
                      f"{pairs} active block pairs, {dt:.2f} s on {threads} threads ({os.cpu_count()} logical cores)"}


def run_reference_arm(args, rank, world):
    if rank != 0:
        return
    threads = use_all_host_threads()
    times, pairs = [], 0
    for i in range(args.warmup + args.steps):
        dt, pairs = cpu_sample_run(args.seq, args.keep, 1, seed=1234 + i)
        if i >= args.warmup:
            times.append(dt)
    ms = 1e3 * sum(times) / len(times)
    val = pairs * FLOPS_PER_PAIR / (ms / 1e3) / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"C3 dynamic random block-sparse, B=1 H={args.heads} S={args.seq} D=128 qb=kb=384 keep={args.keep}; "
                               "each step is a bounded sample: 1 query block of 1 head against all keys"},
        "cpu_baseline": {"value": val, "unit": "TFLOPS", "cores": threads, "kind": "port",
                         "sample": f"torch dense-masked SDPA fwd+bwd (the reference's oracle path; its CUDA kernels are sm_90a-only and "
                                   f"their ThunderKittens dependency is absent), 1 query block x {args.seq} keys per step, {threads} threads"},
        "e2e": {"value": val, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch.distributed as dist
    import flex_block_attn_b200 as fba
    from flex_block_attn_b200 import _cabi, masks
    from flex_block_attn_b200.dist import head_shard

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the operator)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    lib = _cabi.lib()

    S, H, keep = args.seq, args.heads, args.keep
    hs = head_shard(H, world, rank)
    Hl = hs.stop - hs.start
    nb = S // KB
    gen = torch.Generator().manual_seed(1000 + rank)
    shape = (1, Hl, S, D)
    host = [torch.randn(shape, generator=gen).to(torch.bfloat16).pin_memory() for _ in range(4)]
    q, k, v, do = (t.to(dev) for t in host)

    def make_mask(step):
        return masks.bernoulli_mask(1, Hl, nb, nb, keep, seed=7919 * (rank + 1) + step, device=dev)

    def step_resident(step, hook=None):
        mask = make_mask(step)
        lists = fba.build_lists(mask, QB, KB, S, S, need_bwd=True)
        o, lse = fba.forward_with_lists(q, k, v, lists)
        if hook is not None:
            lib.fba_set_timing_events(2, hook[0].cuda_event, hook[1].cuda_event)
        out = fba.backward_with_lists(q, k, v, o, lse, do, lists)
        if hook is not None:
            lib.fba_set_timing_events(0, None, None)
        return mask, out

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    # ---------------------------------------------------------------- device-resident timing
    # One-time set-up that is not a step: first-call initialisation (module load, shared-memory
    # attribute, tensor-map encoder lookup) and growth of torch's caching allocator to the working
    # set, so that the W warm-up steps and the K timed steps all run in steady state.
    for i in range(2):
        step_resident(-1 - i)
    torch.cuda.synchronize()
    for i in range(args.warmup):
        step_resident(i)
    hooks = []
    for _ in range(args.steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); b.record()
        hooks.append((a, b))
    nnz = 0
    sampler = ClockSampler(physical_gpu_index(local_rank))
    barrier()
    if rank == 0:
        sampler.start()
    launches0 = lib.fba_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    masks_seen = []
    for i in range(args.steps):
        m, _ = step_resident(args.warmup + i, hooks[i])
        masks_seen.append(m)
    e1.record()
    barrier()
    launches = lib.fba_launch_count() - launches0
    fba.check_status(dev)
    ms_local = e0.elapsed_time(e1) / args.steps
    ms = max_over_ranks(ms_local)
    nnz_local = sum(int(m.sum().item()) for m in masks_seen) / args.steps
    nnz = sum_over_ranks(nnz_local)
    value = nnz * FLOPS_PER_PAIR / (ms / 1e3) / 1e12
    bwd_ms = statistics.mean(a.elapsed_time(b) for a, b in hooks)
    del masks_seen

    # forward main kernel alone, a few extra steps (reported beside the roofline object)
    fwd_ms = None
    try:
        lists = fba.build_lists(make_mask(0), QB, KB, S, S, need_bwd=False)
        fa, fb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        fa.record(); fb.record()
        lib.fba_set_timing_events(1, fa.cuda_event, fb.cuda_event)
        ts = []
        for _ in range(3):
            fba.forward_with_lists(q, k, v, lists)
            torch.cuda.synchronize()
            ts.append(fa.elapsed_time(fb))
        lib.fba_set_timing_events(0, None, None)
        fwd_ms = statistics.mean(ts)
    except Exception:
        lib.fba_set_timing_events(0, None, None)

    # ---------------------------------------------------------------- end to end through the API
    e2e = None
    if not args.no_e2e:
        copy_stream = torch.cuda.Stream(dev)
        # Two sets of device input buffers: while step s computes on one set, the inputs of step
        # s+1 are copied from pinned host memory into the other (every step's copy is inside the
        # timed region; the first step's copy is fully exposed).
        bufsets = [[torch.empty(shape, dtype=torch.bfloat16, device=dev) for _ in range(4)] for _ in range(2)]
        set_free = [None, None]     # event: compute that last read this set has finished
        set_ready = [None, None]    # events: (q,k,v copied, dO copied)
        result_host = torch.empty(4, dtype=torch.float32).pin_memory()

        def issue_copy(slot):
            with torch.cuda.stream(copy_stream):
                if set_free[slot] is not None:
                    copy_stream.wait_event(set_free[slot])
                for i in range(3):
                    bufsets[slot][i].copy_(host[i], non_blocking=True)
                qkv = torch.cuda.Event(); qkv.record(copy_stream)
                bufsets[slot][3].copy_(host[3], non_blocking=True)
                do = torch.cuda.Event(); do.record(copy_stream)
            set_ready[slot] = (qkv, do)

        def run_e2e(first_step, n):
            cur = torch.cuda.current_stream(dev)
            copy_stream.wait_stream(cur)
            seen = []
            issue_copy(0)
            for j in range(n):
                slot = j & 1
                if j + 1 < n:
                    issue_copy(slot ^ 1)
                bufs = bufsets[slot]
                mask = make_mask(first_step + j)
                cur.wait_event(set_ready[slot][0])
                qq, kk, vv = (b.detach().requires_grad_() for b in bufs[:3])
                o = fba.flex_block_attn_func(qq, kk, vv, QB, KB, mask)
                cur.wait_event(set_ready[slot][1])
                o.backward(bufs[3])
                res = torch.stack([t.sum(dtype=torch.float32) for t in (o.detach(), qq.grad, kk.grad, vv.grad)])   # one read pass each
                result_host.copy_(res, non_blocking=True)
                ev = torch.cuda.Event(); ev.record(cur)
                set_free[slot] = ev
                seen.append(mask)
            return seen

        run_e2e(0, max(2, min(args.warmup, 3)))
        barrier()
        n_e2e = max(2, min(args.steps, 10))
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        ms_seen = run_e2e(100, n_e2e)
        t1.record()
        barrier()
        e_ms = max_over_ranks(t0.elapsed_time(t1) / n_e2e)
        e_nnz = sum_over_ranks(sum(int(m.sum().item()) for m in ms_seen) / n_e2e)
        e2e = {"value": e_nnz * FLOPS_PER_PAIR / (e_ms / 1e3) / 1e12, "unit": "TFLOPS",
               "h2d_bytes_per_step": int(4 * host[0].numel() * 2 * world), "d2h_bytes_per_step": int(16 * world),
               "ms_per_step": e_ms, "steps": n_e2e,
               "note": "q,k,v,dO copied from pinned host memory every step (double-buffered: the copy for step s+1 overlaps the "
                       "compute of step s; the first copy is exposed), flex_block_attn_func + backward through autograd, "
                       "4-float checksum of o,dq,dk,dv read back every step"}
        fba.check_status(dev)

    clocks = sampler.stop() if rank == 0 else None   # sampled over the resident and the end-to-end regions
    total_launches = sum_over_ranks(float(launches))
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = measured_peaks()
    bwd_flops = nnz_local * FLOPS_PER_PAIR_BWD
    achieved = bwd_flops / (bwd_ms / 1e3) / 1e12
    roofline = {
        "kernel": "fba_bwd_kernel", "bound": "tensor", "achieved": achieved, "peak": peaks["sustained"], "unit": "TFLOP/s",
        "frac": achieved / peaks["sustained"], "peak_kind": f"bf16_tflops_sustained of {peaks['source']} (kernel timed inside a long step)",
        "frac_of_burst_peak": achieved / peaks["burst"], "burst_peak": peaks["burst"],
        "ms_per_launch": bwd_ms, "flops_per_launch": bwd_flops,
        "traffic": (BWD_DRAM_BYTES_PER_PAIR * nnz_local) if BWD_DRAM_BYTES_PER_PAIR else None,
        "traffic_note": "bytes per launch, scaled per active pair from the ncu capture of a smaller case (profiles/)",
        "share_of_step": bwd_ms / ms_local,
    }
    if fwd_ms:
        fwd_ach = nnz_local * FLOPS_PER_PAIR_FWD / (fwd_ms / 1e3) / 1e12
        roofline["fwd_kernel"] = {"kernel": "fba_fwd_kernel", "ms_per_launch": fwd_ms, "achieved": fwd_ach,
                                  "frac": fwd_ach / peaks["sustained"], "frac_of_burst_peak": fwd_ach / peaks["burst"]}
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": f"C3 dynamic random block-sparse fwd+bwd, B=1 H={H} S={S} D=128 q_block=kv_block=384 "
                               f"Bernoulli(keep={keep})|diag per-(b,h) mask; mask draw + compaction inside the step; "
                               f"heads split {Hl}/GPU", "l2": "inputs (4 x %.0f MB per rank) exceed the 126 MB L2" % (q.numel() * 2 / 1e6),
                   "active_block_pairs": nnz, "pct_of_measured_burst_peak": 100 * value / (peaks["burst"] * world),
                   "pct_of_measured_sustained_peak": 100 * value / (peaks["sustained"] * world),
                   "pct_of_nominal_2250": 100 * value / (2250.0 * world)},
        "e2e": e2e, "gpu_launches": int(total_launches), "clocks": clocks, "roofline": roofline,
    }
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(S, keep)
    if world > 1:
        dist.destroy_process_group()
    print(json.dumps(line), flush=True)   # last line of stdout


if __name__ == "__main__":
    main()
