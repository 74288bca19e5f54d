"""Benchmark of the block-sparse attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c3|c2|c4|c5] [--dq-mode atomic|qmajor]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" = one pass of the hot path over one batch of synthetic input: build the block mask /
index lists on the device, forward, backward.  The default workload (c3) is the one the metric is
quoted on: dynamic random block-sparse attention, B=1, H=24, D=128, q_block=kv_block=384, S=69120,
Bernoulli(keep 0.4) per-(batch, head) mask with the diagonal forced on, q,k,v,dO ~ N(0,1) bf16 from
a seed.  The other benchmark configurations run through the same code with --workload:
  c2  full attention, S=30720, 384-blocks, inputs N(0,1)*0.5
  c4  3-D sliding-tile attention over 3x6x10 tiles of 384 tokens (S=69120), lists built without a mask
  c5  SSTA (STA window + top-8 pooled q.k), q_block 128 / kv_block 384, B=2, S=69120
With N GPUs the 24 heads are split evenly over the ranks (no data-path collective; strong scaling:
total work is fixed).

The printed line carries
  value      whole-job effective TFLOPS (14*qb*kb*D FLOPs per active block pair, active blocks
             only), inputs resident in HBM, CUDA events, max over ranks;
  e2e        the same metric through the public API (flex_block_attn_func + backward) with q, k, v,
             dO copied from pinned host memory and O, dQ, dK, dV copied back to pinned host memory
             inside the timed region (e2e_checksum_only: reading back a 4-float checksum instead);
  roofline   the backward main kernel (largest share of the step) against the measured dense
             bf16 peak, timed live with CUDA events recorded around that kernel alone;
  cpu_baseline  torch dense-masked SDPA (the reference's own oracle path) on the host cores, on a
             bounded sample of the same workload;
and, with N > 1 (default workload only),
  multi_gpu_check  a small sequence-sharded problem through both Ulysses paths (NCCL exchange and
             the fused peer-memory exchange) compared with the same rank computing it alone;
  c5         configuration 5 with inputs arriving sequence-sharded: the sequence<->head exchange
             timed on its own, beside mask/list building, forward and backward, for both paths.
`--impl reference` times only the CPU path (the reference's CUDA kernels are Hopper-only and
their ThunderKittens dependency is not vendored, so they cannot run on this machine).
"""
from __future__ import annotations

import argparse
import json
import os
import re
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

D = 128
METRIC = "fwd+bwd effective TFLOPS (active blocks), S=69120 sparse 0.6; % B200 bf16 peak"
STA_GRID = (3, 6, 10)          # tiles of 6x8x8 = 384 tokens over the 18x48x80 latent grid
LATENT_GRID = (18, 48, 80)
LATENT_TILE = (6, 8, 8)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=["c3", "c2", "c4", "c5"], default="c3")
    ap.add_argument("--seq", type=int, default=None, help="sequence length (c3 sweep: 11520 ... 69120)")
    ap.add_argument("--heads", type=int, default=24)
    ap.add_argument("--keep", type=float, default=0.4)
    ap.add_argument("--dq-mode", choices=["atomic", "qmajor"], default=None,
                    help="dQ strategy of the backward (default: the library's default)")
    ap.add_argument("--fp8", action="store_true",
                    help="also time the inference forward over an e4m3 key/value cache (reported as fp8_fwd)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-multi-gpu-extras", action="store_true",
                    help="skip multi_gpu_check and the sequence-sharded c5 object at N > 1")
    return ap.parse_args()


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"burst": float(d["bf16_tflops"]), "sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"burst": 1590.0, "sustained": 1400.0, "source": "fallback"}


def bwd_dram_bytes_per_pair():
    """DRAM traffic of the backward main kernel per active 384x384 block pair, read from the committed
    ncu summary (its `dram_bytes_per_active_pair = N` line); None if the summary does not carry one."""
    best = None
    for f in sorted((ROOT / "profiles").glob("fba_bwd_kernel_*.md")):
        m = re.search(r"dram_bytes_per_active_pair\s*=\s*([0-9.eE+]+)", f.read_text())
        if m:
            best = (float(m.group(1)), f.name)
    return best


class ClockSampler:
    """nvidia-smi clock / throttle-reason sampling (read-only query), one process for the whole run.

    The process is started long before the first timed region -- its start-up (NVML attaching to every
    GPU of the machine) takes driver locks that stall kernel launches for a few hundred milliseconds --
    and every sample carries a timestamp, so that a timed region is summarised afterwards from the
    samples that fall between its begin() and end() marks."""

    FIELDS = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None
        self.windows = {}
        self.rows = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def begin(self, name):
        self.windows[name] = [time.time(), None]

    def end(self, name):
        self.windows[name][1] = time.time()

    def stop(self):
        if self.proc is None or self.rows is not None:
            return
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        import datetime

        self.rows = []
        try:
            for line in Path(self.path).read_text().splitlines():
                parts = [x.strip() for x in line.split(",")]
                if len(parts) < 10:
                    continue
                try:
                    t = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    self.rows.append((t, float(parts[2]), float(parts[3]), parts[4], parts[6:10]))
                except ValueError:
                    continue
            os.unlink(self.path)
        except Exception:
            pass

    def summary(self, name):
        """Median SM clock, maximum clock, throttle reasons and median power over one window."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.stop()
        t0, t1 = self.windows[name]
        rows = [r for r in self.rows if t0 <= r[0] <= t1]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no_samples"]}
        reasons = set()
        for r in rows:
            for nm, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        out = {"sm_mhz": statistics.median(r[1] for r in rows), "sm_max_mhz": max(r[2] for r in rows),
               "reasons": sorted(reasons), "samples": len(rows)}
        pw = []
        for r in rows:
            try:
                pw.append(float(r[3]))
            except ValueError:
                pass
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
# Workloads
# ------------------------------------------------------------------------------------------------
class Workload:
    """One benchmark configuration for the heads of one rank: shapes, input scale and the per-step
    construction of the index lists (the "mask creation" that the step includes)."""

    def __init__(self, name, args, Hl, rank, dev):
        self.name, self.Hl, self.rank, self.dev = name, Hl, rank, dev
        self.scale = 1.0
        self.B = 1
        if name == "c2":
            self.S, self.qb, self.kb = args.seq or 30720, 384, 384
            self.scale = 0.5
            self.desc = f"C2 full attention fwd+bwd, B=1 H={args.heads} S={self.S} D=128 q_block=kv_block=384, all-ones 2-D mask"
        elif name == "c3":
            self.S, self.qb, self.kb = args.seq or 69120, 384, 384
            self.keep = args.keep
            self.desc = (f"C3 dynamic random block-sparse fwd+bwd, B=1 H={args.heads} S={self.S} D=128 q_block=kv_block=384 "
                         f"Bernoulli(keep={args.keep})|diag per-(b,h) mask")
        elif name == "c4":
            self.S, self.qb, self.kb = 69120, 384, 384
            self.desc = f"C4 sliding-tile attention fwd+bwd, B=1 H={args.heads} S=69120 D=128, 3x6x10 tiles of 384 tokens, window 3x3x3"
        else:
            self.B = 2
            self.S, self.qb, self.kb = 69120, 128, 384
            self.desc = (f"C5 SSTA (STA 3x3x3 window + top-8 pooled q.k) fwd+bwd, B=2 H={args.heads} S=69120 D=128 "
                         "q_block=128 kv_block=384, per-(b,h) mask [540,180]")
        self.flops_fwd = 4 * self.qb * self.kb * D
        self.flops_bwd = 10 * self.qb * self.kb * D
        self.flops = self.flops_fwd + self.flops_bwd
        self.shape = (self.B, Hl, self.S, D)

    def lists(self, fba, masks, step, q, k):
        """-> (SparseLists, mask-or-None, active block pairs on this rank as a 0-d device tensor or int)."""
        if self.name == "c2":
            m = masks.full_mask(self.S // self.qb, self.S // self.kb, device=self.dev)
            return fba.build_lists(m, self.qb, self.kb, self.S, self.S, need_bwd=True), m, m.numel() * self.B * self.Hl
        if self.name == "c3":
            nb = self.S // self.qb
            m = masks.bernoulli_mask(1, self.Hl, nb, nb, self.keep, seed=7919 * (self.rank + 1) + step, device=self.dev)
            return fba.build_lists(m, self.qb, self.kb, self.S, self.S, need_bwd=True), m, m.sum()
        if self.name == "c4":
            l = fba.sta_lists(STA_GRID, (1, 1, 1), tile_tokens=384, device=self.dev)
            return l, None, l.fwd_cnt.sum() * (self.B * self.Hl)
        l, m = fba.ssta_lists(q, k, STA_GRID, self.qb, self.kb, topk=8)
        return l, m, m.sum()


# ------------------------------------------------------------------------------------------------
# CPU path (the reference's torch oracle) on a bounded sample of the workload
# ------------------------------------------------------------------------------------------------
QB_CPU = KB_CPU = 384
FLOPS_PER_PAIR_CPU = 14 * QB_CPU * KB_CPU * D


def cpu_sample_run(S: int, keep: float, n_qblocks: int, seed: int = 1234):
    """fwd+bwd of `n_qblocks` query blocks of one head against all S keys; returns (seconds, pairs)."""
    from oracle import dense_oracle as orc

    g = torch.Generator().manual_seed(seed)
    nb = S // KB_CPU
    q = torch.randn((1, 1, n_qblocks * QB_CPU, D), generator=g).requires_grad_()
    k = torch.randn((1, 1, S, D), generator=g).requires_grad_()
    v = torch.randn((1, 1, S, D), generator=g).requires_grad_()
    do = torch.randn((1, 1, n_qblocks * QB_CPU, D), generator=g)
    mask = torch.rand((n_qblocks, nb), generator=g) < keep
    mask[torch.arange(n_qblocks), torch.arange(n_qblocks)] = True
    t0 = time.perf_counter()
    o = orc.sdpa_dense(q, k, v, mask, QB_CPU, KB_CPU)
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
    nq = 8 if S >= 8 * QB_CPU else max(1, S // QB_CPU)
    dt, pairs = cpu_sample_run(S, keep, nq)
    reps = max(1, min(24, int(round(target_s / max(dt, 1e-3)))))
    for r in range(1, reps):
        d, p = cpu_sample_run(S, keep, nq, seed=1234 + r)
        dt += d
        pairs += p
    tflops = pairs * FLOPS_PER_PAIR_CPU / dt / 1e12
    return {"value": tflops, "unit": "TFLOPS", "cores": threads, "kind": "port",
            "sample": f"torch F.scaled_dot_product_attention + dense token mask (the reference's oracle path), fp32, "
                      f"fwd+bwd of {reps} x {nq} query blocks of one head against all {S} keys of the S={S} keep={keep} workload, "
                      f"{pairs} active block pairs, {dt:.2f} s on {threads} threads ({os.cpu_count()} logical cores)"}


def run_reference_arm(args, rank, world):
    if rank != 0:
        return
    threads = use_all_host_threads()
    S = args.seq or 69120
    times, pairs = [], 0
    for i in range(args.warmup + args.steps):
        dt, pairs = cpu_sample_run(S, args.keep, 1, seed=1234 + i)
        if i >= args.warmup:
            times.append(dt)
    ms = 1e3 * sum(times) / len(times)
    val = pairs * FLOPS_PER_PAIR_CPU / (ms / 1e3) / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"C3 dynamic random block-sparse, B=1 H={args.heads} S={S} D=128 qb=kb=384 keep={args.keep}; "
                               "each step is a bounded sample: 1 query block of 1 head against all keys"},
        "cpu_baseline": {"value": val, "unit": "TFLOPS", "cores": threads, "kind": "port",
                         "sample": f"torch dense-masked SDPA fwd+bwd (the reference's oracle path; its CUDA kernels are sm_90a-only and "
                                   f"their ThunderKittens dependency is absent), 1 query block x {S} keys per step, {threads} threads"},
        "e2e": {"value": val, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# Multi-GPU extras (N > 1): correctness of both Ulysses paths, and configuration 5 sequence-sharded
# ------------------------------------------------------------------------------------------------
def _close(got, want, max_abs=1e-2, min_cos=0.9995):
    g, w = got.float().flatten().double(), want.float().flatten().double()
    ma = (g - w).abs().max().item()
    cos = (g @ w).item() / max((g.norm() * w.norm()).item(), 1e-30)
    return ma <= max_abs * max(1.0, w.abs().max().item()) and cos >= min_cos, ma, cos


def multi_gpu_check(fba, fd, masks, dist, dev, rank, world):
    """A small sequence-sharded problem (B=2, H=8, S=3072, q_block 128 / kv_block 384, SSTA mask)
    through ulysses_flex_block_attn (NCCL exchange) and ulysses_tile_major_attn (fused peer-memory
    exchange), each against this rank computing the whole problem alone: O, dK, dV bit for bit, dQ
    (fp32 reductions in arrival order) by value."""
    B, H, qb, kb = 2, 8, 128, 384
    grid, tile = (2, 8, 192), (2, 8, 24)                 # S = 3072 tokens, 8 tiles of 384
    tile_grid = (1, 1, 8)
    S = grid[0] * grid[1] * grid[2]
    Sl, Hl = S // world, H // world
    sl, hs = slice(rank * Sl, (rank + 1) * Sl), slice(rank * Hl, (rank + 1) * Hl)
    g = torch.Generator().manual_seed(4242)              # same seed on every rank: same full problem
    raster = [torch.randn((B, S, H, D), generator=g).to(torch.bfloat16).to(dev) for _ in range(4)]   # q k v dO
    tm = lambda t: masks.to_tile_major(t.contiguous(), grid, tile)       # [B, H, S, D] tile-major
    rs = lambda t: masks.from_tile_major(t.contiguous(), grid, tile)     # [B, S, H, D] raster

    def mask_fn(qh, kh):
        return masks.ssta_mask(qh, kh, tile_grid, qb, kb, topk=2)

    out = {}
    # whole problem on this rank alone
    full = [tm(t) for t in raster]
    qf, kf, vf = (t.clone().requires_grad_() for t in full[:3])
    of = fba.flex_block_attn_func(qf, kf, vf, qb, kb, mask_fn(qf, kf))
    of.backward(full[3])
    torch.cuda.synchronize()

    def verdict(name, o, dq, dk, dv, want):
        bad = []
        for nm, g_, w_, exact in (("O", o, want[0], True), ("dK", dk, want[2], True), ("dV", dv, want[3], True),
                                  ("dQ", dq, want[1], False)):
            if exact:
                if not torch.equal(g_, w_):
                    bad.append(f"{nm} differs (max {(g_.float() - w_.float()).abs().max().item():.3g})")
            else:
                ok, ma, cos = _close(g_, w_)
                if not ok:
                    bad.append(f"{nm} max_abs {ma:.3g} cos {cos:.6f}")
        t = torch.tensor([len(bad)], device=dev)
        dist.all_reduce(t)
        out[name] = "ok" if int(t.item()) == 0 else ("rank %d: %s" % (rank, "; ".join(bad)) if bad else "failed on another rank")

    try:
        ql, kl, vl = (t[:, :, sl].contiguous().requires_grad_() for t in full[:3])
        o = fd.ulysses_flex_block_attn(ql, kl, vl, qb, kb, mask_fn)
        o.backward(full[3][:, :, sl].contiguous())
        torch.cuda.synchronize()
        verdict("nccl_ulysses", o.detach(), ql.grad, kl.grad, vl.grad,
                (of.detach()[:, :, sl], qf.grad[:, :, sl], kf.grad[:, :, sl], vf.grad[:, :, sl]))
    except Exception as e:   # reported in the line; the run then exits non-zero
        out["nccl_ulysses"] = f"{type(e).__name__}: {e}"
    try:
        ex = fd.PeerExchange(B, H, grid, tile, slots=4)
        try:
            q2, k2, v2 = (t[:, sl].contiguous().requires_grad_() for t in raster[:3])
            o2 = fd.ulysses_tile_major_attn(q2, k2, v2, qb, kb, mask_fn, ex)
            o2.backward(raster[3][:, sl].contiguous())
            torch.cuda.synchronize()
            verdict("peer_exchange", o2.detach(), q2.grad, k2.grad, v2.grad,
                    (rs(of.detach())[:, sl], rs(qf.grad)[:, sl], rs(kf.grad)[:, sl], rs(vf.grad)[:, sl]))
        finally:
            ex.close()
    except Exception as e:
        out["peer_exchange"] = f"{type(e).__name__}: {e}"
    fba.check_status(dev)
    return out


def c5_sequence_sharded(fba, fd, masks, dist, dev, rank, world, reps=3):
    """Configuration 5 with inputs arriving sequence-sharded over the ranks (B=2, H=24, S=69120,
    q_block 128 / kv_block 384, SSTA mask built after the exchange).  Every phase is timed on its
    own with CUDA events (median of `reps`, max over ranks): the exchange towards the heads (q, k, v,
    dO), mask + list building, forward, backward, the exchange back (O, dQ, dK, dV)."""
    B, H, qb, kb = 2, 24, 128, 384
    S = LATENT_GRID[0] * LATENT_GRID[1] * LATENT_GRID[2]
    Sl, Hl = S // world, H // world
    flops_pair = 14 * qb * kb * D
    g = torch.Generator().manual_seed(9000 + rank)
    mk = lambda shape: torch.randn(shape, generator=g).to(torch.bfloat16).to(dev)
    bytes_tensor = B * Sl * H * D * 2                      # one local tensor
    leaving = bytes_tensor * (world - 1) // world

    def timed(fn):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        r = fn()
        b.record()
        return r, (a, b)

    def reduce_ms(evs):
        torch.cuda.synchronize()
        t = torch.tensor([statistics.median(a.elapsed_time(b) for a, b in evs)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def run(path, to_head, to_seq, local):
        phases = {k_: [] for k_ in ("a2a_in", "mask_lists", "fwd", "bwd", "a2a_out")}
        pairs = None
        for _ in range(reps + 1):                          # first pass warms up
            dist.barrier()
            heads, ev = timed(lambda: [to_head(t, i) for i, t in enumerate(local)])
            phases["a2a_in"].append(ev)
            qh, kh, vh, doh = heads
            (lists, mask), ev = timed(lambda: fba.ssta_lists(qh, kh, STA_GRID, qb, kb, topk=8))
            phases["mask_lists"].append(ev)
            (o, lse), ev = timed(lambda: fba.forward_with_lists(qh, kh, vh, lists))
            phases["fwd"].append(ev)
            grads, ev = timed(lambda: fba.backward_with_lists(qh, kh, vh, o, lse, doh, lists))
            phases["bwd"].append(ev)
            _, ev = timed(lambda: [to_seq(t, i) for i, t in enumerate((o,) + tuple(grads))])
            phases["a2a_out"].append(ev)
            pairs = mask.sum()
        ms = {k_: reduce_ms(v[1:]) for k_, v in phases.items()}
        t = pairs.to(torch.float64).reshape(1)
        dist.all_reduce(t)
        total_pairs = float(t.item())
        kern = ms["fwd"] + ms["bwd"]
        allms = sum(ms.values())
        return {"a2a_in_ms": ms["a2a_in"], "a2a_out_ms": ms["a2a_out"], "mask_lists_ms": ms["mask_lists"], "fwd_ms": ms["fwd"],
                "bwd_ms": ms["bwd"], "a2a_bytes_leaving_gpu_per_direction": 4 * leaving,
                "a2a_in_gbs_per_gpu": 4 * leaving / (ms["a2a_in"] / 1e3) / 1e9,
                "a2a_out_gbs_per_gpu": 4 * leaving / (ms["a2a_out"] / 1e3) / 1e9,
                "tflops_kernels_only": total_pairs * flops_pair / (kern / 1e3) / 1e12,
                "tflops_with_exchange_and_mask": total_pairs * flops_pair / (allms / 1e3) / 1e12,
                "active_block_pairs": total_pairs}

    out = {"workload": f"C5 SSTA B=2 H=24 S={S} D=128 q_block=128 kv_block=384, inputs sequence-sharded [2, {Sl}, 24, 128] per GPU",
           "timing": f"CUDA events per phase, median of {reps} after 1 warm-up pass, max over ranks; phases run back to back on one stream"}
    try:
        # NCCL path: head-major, tile-major chunks [B, H, S/P, D] exchanged by grouped send/recv
        local = [mk((B, H, Sl, D)) for _ in range(4)]
        out["nccl"] = run("nccl", lambda t, i: fd.seq_to_head(t), lambda t, i: fd.head_to_seq(t), local)
        del local
    except Exception as e:
        out["nccl"] = {"error": f"{type(e).__name__}: {e}"}
    torch.cuda.empty_cache()
    try:
        # fused path: native [B, S/P, H, D] raster chunks; one kernel does transpose + tile-major
        # reorder + the exchange by peer stores over NVLink
        ex = fd.PeerExchange(B, H, LATENT_GRID, LATENT_TILE, slots=4)
        try:
            local = [mk((B, Sl, H, D)) for _ in range(4)]
            out["peer_exchange"] = run("peer", lambda t, i: ex.seq_to_head(t, i), lambda t, i: ex.head_to_seq(t, i), local)
            out["peer_exchange"]["note"] = ("includes the [B,S,H,D] raster -> [B,H,S,D] tile-major layout change, which the NCCL "
                                            "path's inputs have already had")
        finally:
            ex.close()
    except Exception as e:
        out["peer_exchange"] = {"error": f"{type(e).__name__}: {e}"}
    fba.check_status(dev)
    torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------------------------------
def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    if args.dq_mode:
        os.environ["FBA_DQ_MODE"] = args.dq_mode
    if world > 1:
        # the fused exchange stores into peer memory with plain st.global; NVLS multicast is not used
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")

    import torch.distributed as dist
    import flex_block_attn_b200 as fba
    from flex_block_attn_b200 import _cabi, masks
    from flex_block_attn_b200 import dist as fd

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the operator)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    lib = _cabi.lib()

    H = args.heads
    hs = fd.head_shard(H, world, rank)
    Hl = hs.stop - hs.start
    wl = Workload(args.workload, args, Hl, rank, dev)
    gen = torch.Generator().manual_seed(1000 + rank)
    shape = wl.shape
    host = [(torch.randn(shape, generator=gen) * wl.scale).to(torch.bfloat16).pin_memory() for _ in range(4)]
    q, k, v, do = (t.to(dev) for t in host)

    def step_resident(step, hook=None):
        lists, _, pairs = wl.lists(fba, masks, step, q, k)
        o, lse = fba.forward_with_lists(q, k, v, lists)
        if hook is not None:
            lib.fba_set_timing_events(2, hook[0].cuda_event, hook[1].cuda_event)
        out = fba.backward_with_lists(q, k, v, o, lse, do, lists)
        if hook is not None:
            lib.fba_set_timing_events(0, None, None)
        return pairs, out

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
    sampler = ClockSampler(physical_gpu_index(local_rank))
    if rank == 0:
        sampler.start()
    # (`keep` holds a step's outputs until the next step has produced its own, exactly as the timed
    # loop does: with a shorter lifetime here the timed loop's peak would be higher than the warm-up's
    # and the allocator would call cudaMalloc -- a device-wide synchronisation -- inside the timed region.)
    keep = None
    for i in range(2):
        keep = step_resident(-1 - i)
    torch.cuda.synchronize()
    for i in range(args.warmup):
        keep = step_resident(i)
    hooks = []
    for _ in range(args.steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); b.record()
        hooks.append((a, b))
    barrier()
    sampler.begin("resident")
    launches0 = lib.fba_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    pairs_seen = []
    for i in range(args.steps):
        keep = step_resident(args.warmup + i, hooks[i])
        pairs_seen.append(keep[0])
    e1.record()
    barrier()
    sampler.end("resident")
    launches = lib.fba_launch_count() - launches0
    fba.check_status(dev)
    ms_local = e0.elapsed_time(e1) / args.steps
    ms = max_over_ranks(ms_local)
    nnz_local = sum(float(p) for p in pairs_seen) / args.steps
    nnz = sum_over_ranks(nnz_local)
    value = nnz * wl.flops / (ms / 1e3) / 1e12
    bwd_ms = statistics.mean(a.elapsed_time(b) for a, b in hooks)
    del pairs_seen, keep

    # forward main kernel alone, a few extra steps (reported beside the roofline object)
    fwd_ms = None
    try:
        lists, _, _ = wl.lists(fba, masks, 0, q, k)
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
        del lists
    except Exception:
        lib.fba_set_timing_events(0, None, None)

    # mask draw + compaction (both directions) + work orders, timed alone (it is inside every step)
    lists_ms = None
    try:
        evs = []
        for i in range(6):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            l, _, _ = wl.lists(fba, masks, 1000 + i, q, k)
            l.fwd_list(ordered=True)
            l.bwd_list(Hl, Hl)
            b.record()
            evs.append((a, b))
        torch.cuda.synchronize()
        lists_ms = statistics.median(a.elapsed_time(b) for a, b in evs[1:])
        del l
    except Exception:
        pass

    # inference forward over an e4m3 key / value cache, same lists (optional)
    fp8_fwd = None
    if args.fp8:
        cache = fba.quantize_kv(k, v, wl.kb)
        lists, _, pairs = wl.lists(fba, masks, 0, q, k)
        fa, fb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        fa.record(); fb.record()
        lib.fba_set_timing_events(1, fa.cuda_event, fb.cuda_event)
        ts8, ts16 = [], []
        for _ in range(5):
            fba.flex_block_attn_fp8kv(q, cache, wl.qb, wl.kb, lists)
            torch.cuda.synchronize()
            ts8.append(fa.elapsed_time(fb))
            fba.forward_with_lists(q, k, v, lists, need_lse=False)
            torch.cuda.synchronize()
            ts16.append(fa.elapsed_time(fb))
        lib.fba_set_timing_events(0, None, None)
        t8, t16 = statistics.median(ts8[1:]), statistics.median(ts16[1:])
        fl = float(pairs) * wl.flops_fwd
        fp8_fwd = {"ms_fp8": t8, "ms_bf16": t16, "tflops_fp8": fl / (t8 / 1e3) / 1e12, "tflops_bf16": fl / (t16 / 1e3) / 1e12,
                   "note": "forward kernel alone (CUDA events around it), this rank's heads, median of 4; K/V cache in e4m3 with "
                           f"one scale per {wl.kb} keys, q quantised in the kernel"}
        del cache, lists

    # ---------------------------------------------------------------- end to end through the API
    e2e = None
    e2e_checksum = None
    if not args.no_e2e:
        sampler.begin("e2e")
        copy_stream = torch.cuda.Stream(dev)
        back_stream = torch.cuda.Stream(dev)
        # Two sets of device input buffers: while step s computes on one set, the inputs of step
        # s+1 are copied from pinned host memory into the other (every step's copy is inside the
        # timed region; the first step's copy is fully exposed).  The results of step s travel back
        # to pinned host memory on a third stream while step s+1 computes; the last step's copy
        # back is exposed, and the timed region ends only when it has landed.
        bufsets = [[torch.empty(shape, dtype=torch.bfloat16, device=dev) for _ in range(4)] for _ in range(2)]
        set_free = [None, None]     # event: compute that last read this set has finished
        set_ready = [None, None]    # events: (q,k,v copied, dO copied)
        result_host = torch.empty(4, dtype=torch.float32).pin_memory()
        results_host = [torch.empty(shape, dtype=torch.bfloat16).pin_memory() for _ in range(4)]

        def issue_copy(slot):
            with torch.cuda.stream(copy_stream):
                if set_free[slot] is not None:
                    copy_stream.wait_event(set_free[slot])
                for i in range(3):
                    bufsets[slot][i].copy_(host[i], non_blocking=True)
                qkv = torch.cuda.Event(); qkv.record(copy_stream)
                bufsets[slot][3].copy_(host[3], non_blocking=True)
                dov = torch.cuda.Event(); dov.record(copy_stream)
            set_ready[slot] = (qkv, dov)

        def run_e2e(first_step, n, full_results):
            cur = torch.cuda.current_stream(dev)
            copy_stream.wait_stream(cur)
            back_stream.wait_stream(cur)
            seen = []
            issue_copy(0)
            for j in range(n):
                slot = j & 1
                if j + 1 < n:
                    issue_copy(slot ^ 1)
                bufs = bufsets[slot]
                cur.wait_event(set_ready[slot][0])
                qq, kk, vv = (b.detach().requires_grad_() for b in bufs[:3])
                lists, _, pairs = wl.lists(fba, masks, first_step + j, qq.detach(), kk.detach())
                o = fba.flex_block_attn_func(qq, kk, vv, wl.qb, wl.kb, lists)
                if full_results:       # O is final after the forward: it travels back while the backward runs
                    fwd_done = torch.cuda.Event(); fwd_done.record(cur)
                    with torch.cuda.stream(back_stream):
                        back_stream.wait_event(fwd_done)
                        results_host[0].copy_(o.detach(), non_blocking=True)
                        o.record_stream(back_stream)
                cur.wait_event(set_ready[slot][1])
                o.backward(bufs[3])
                outs = (o.detach(), qq.grad, kk.grad, vv.grad)
                if full_results:
                    done = torch.cuda.Event(); done.record(cur)
                    with torch.cuda.stream(back_stream):
                        back_stream.wait_event(done)
                        for t, h in zip(outs[1:], results_host[1:]):
                            h.copy_(t, non_blocking=True)
                            t.record_stream(back_stream)
                else:
                    res = torch.stack([t.sum(dtype=torch.float32) for t in outs])   # one read pass each
                    result_host.copy_(res, non_blocking=True)
                ev = torch.cuda.Event(); ev.record(cur)
                set_free[slot] = ev
                seen.append(pairs)
            cur.wait_stream(back_stream)    # the timed region includes the last copy back
            return seen

        def measure(full_results):
            run_e2e(0, max(2, min(args.warmup, 3)), full_results)
            barrier()
            n_e2e = max(2, min(args.steps, 20))
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            seen = run_e2e(100, n_e2e, full_results)
            t1.record()
            barrier()
            e_ms = max_over_ranks(t0.elapsed_time(t1) / n_e2e)
            e_nnz = sum_over_ranks(sum(float(p) for p in seen) / n_e2e)
            nbytes = int(4 * host[0].numel() * 2 * world)
            return {"value": e_nnz * wl.flops / (e_ms / 1e3) / 1e12, "unit": "TFLOPS", "h2d_bytes_per_step": nbytes,
                    "d2h_bytes_per_step": nbytes if full_results else int(16 * world), "ms_per_step": e_ms, "steps": n_e2e}

        e2e = measure(True)
        e2e["note"] = ("q,k,v,dO copied from pinned host memory every step (double-buffered: the copy for step s+1 overlaps the "
                       "compute of step s; the first copy is exposed); index lists built on the device; flex_block_attn_func + "
                       "backward through autograd; O,dQ,dK,dV copied back to pinned host memory on a third stream (overlaps the "
                       "next step; the last copy back is exposed and inside the timed region)")
        e2e_checksum = measure(False)
        e2e_checksum["note"] = "same, but a 4-float checksum of O,dQ,dK,dV is read back instead of the tensors"
        fba.check_status(dev)
        del bufsets, results_host
        sampler.end("e2e")

    clocks = clocks_e2e = None
    if rank == 0:
        clocks = sampler.summary("resident")      # the device-resident timed region only
        if "e2e" in sampler.windows:
            clocks_e2e = sampler.summary("e2e")
    total_launches = sum_over_ranks(float(launches))

    # ---------------------------------------------------------------- multi-GPU extras
    mg_check = c5 = None
    if world > 1 and args.workload == "c3" and not args.no_multi_gpu_extras:
        del q, k, v, do, host
        torch.cuda.empty_cache()
        mg_check = multi_gpu_check(fba, fd, masks, dist, dev, rank, world)
        c5 = c5_sequence_sharded(fba, fd, masks, dist, dev, rank, world)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        if mg_check and any(vv != "ok" for vv in mg_check.values()):
            raise SystemExit(3)
        return

    peaks = measured_peaks()
    bwd_flops = nnz_local * wl.flops_bwd
    achieved = bwd_flops / (bwd_ms / 1e3) / 1e12
    traffic = bwd_dram_bytes_per_pair()
    pair_scale = (wl.qb * wl.kb) / (384.0 * 384.0)
    roofline = {
        "kernel": "fba_bwd_kernel", "bound": "tensor", "achieved": achieved, "peak": peaks["sustained"], "unit": "TFLOP/s",
        "frac": achieved / peaks["sustained"], "peak_kind": f"bf16_tflops_sustained of {peaks['source']} (kernel timed inside a long step)",
        "frac_of_burst_peak": achieved / peaks["burst"], "burst_peak": peaks["burst"],
        "ms_per_launch": bwd_ms, "flops_per_launch": bwd_flops,
        "traffic": (traffic[0] * pair_scale * nnz_local) if traffic else None,
        "traffic_note": ("bytes per launch = dram_bytes_per_active_pair of profiles/%s (ncu capture of a smaller case) x the active "
                         "pairs of this launch" % traffic[1]) if traffic else "no ncu summary with a per-pair figure found",
        "share_of_step": bwd_ms / ms_local, "dq_mode": os.environ.get("FBA_DQ_MODE", "atomic"),
    }
    if fwd_ms:
        fwd_ach = nnz_local * wl.flops_fwd / (fwd_ms / 1e3) / 1e12
        roofline["fwd_kernel"] = {"kernel": "fba_fwd_kernel", "ms_per_launch": fwd_ms, "achieved": fwd_ach,
                                  "frac": fwd_ach / peaks["sustained"], "frac_of_burst_peak": fwd_ach / peaks["burst"]}
    per_rank_mb = 4 * shape[0] * shape[1] * shape[2] * shape[3] * 2 / 1e6
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": f"{wl.desc}; mask / list building inside the step; heads split {Hl}/GPU",
                   "l2": ("working set per rank: q,k,v,dO,O,dQ,dK,dV = %.0f MB plus a %.0f MB fp32 dQ accumulator, streamed once per "
                          "step (126 MB L2); no explicit flush between steps" % (2 * per_rank_mb, per_rank_mb / 4 * 2)),
                   "active_block_pairs": nnz, "pct_of_measured_burst_peak": 100 * value / (peaks["burst"] * world),
                   "pct_of_measured_sustained_peak": 100 * value / (peaks["sustained"] * world),
                   "pct_of_nominal_2250": 100 * value / (2250.0 * world),
                   "work_order": os.environ.get("FBA_WORK_ORDER", "1") != "0"},
        "e2e": e2e, "e2e_checksum_only": e2e_checksum, "gpu_launches": int(total_launches), "clocks": clocks,
        "clocks_e2e": clocks_e2e, "roofline": roofline,
    }
    if clocks and clocks.get("sm_mhz"):
        line["per_clock"] = {"tflops_per_gpu_per_ghz": value / world / (clocks["sm_mhz"] / 1e3),
                             "note": "value / n_gpus / median SM clock of rank 0 during the device-resident timed region"}
    line["breakdown_ms"] = {"mask_lists_order": lists_ms, "fwd_kernel_alone": fwd_ms, "bwd_main_kernel_in_step": bwd_ms,
                            "step": ms_local,
                            "note": "mask draw / list building + compaction + work orders timed alone with CUDA events (median of 5); "
                                    "forward kernel alone after the timed loop; backward main kernel inside the timed steps"}
    if fp8_fwd is not None:
        line["fp8_fwd"] = fp8_fwd
    if mg_check is not None:
        line["multi_gpu_check"] = mg_check
    if c5 is not None:
        line["c5"] = c5
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(args.seq or 69120, args.keep)
    if world > 1:
        dist.destroy_process_group()
    print(json.dumps(line), flush=True)   # last line of stdout
    if mg_check and any(vv != "ok" for vv in mg_check.values()):
        raise SystemExit(3)


if __name__ == "__main__":
    main()
