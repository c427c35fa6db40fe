"""Benchmark of the Pairformer / diffusion-transformer hot path on B200.

    python bench.py --gpus 1 --steps K --warmup W            # this repository's sm_100a path (default workload: trunk)
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU path on the host cores
    python bench.py --workload trimul    ...                 # TriangleMultiplication outgoing + incoming, N = 768
    python bench.py --workload diffusion ...                 # 24-block DiffusionTransformer, N = 2048, one sample per GPU

Workload ``trunk`` (the headline): one recycle of the 48-block Pairformer trunk at N = 1024 tokens (bf16, seed-2
random-init weights, synthetic z, s ~ N(0,1) with a random 10 % padding mask).  A step is one recycle.  Prints ONE JSON
line.  ``value`` is ms per recycle with z and s already resident in HBM, timed with the library's per-launch
instrumentation OFF; ``e2e`` is the same recycle called with HOST buffers (pinned host -> device copy of z, s and the
masks, 48 blocks, device -> host copy of the updated z and s inside the timed region).  The per-kernel table comes from
a separate, untimed pass with the instrumentation on.  Inputs (z is 268 MB) are larger than the 126 MB L2, so no flush
is needed between steps.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as ge  # noqa: E402

KERNEL_CLASSES = ["layernorm", "trimul_proj", "trimul_contract", "channel_ln", "linear_gate_resid", "linear",
                  "attention", "linear_swiglu", "mask_bias", "swiglu", "peer_exchange", "apb_attention"]


def flops_block(n, c=128, cs=384):
    tri = 2 * (2 * n ** 3 * c + 12 * n * n * c * c)
    att = 2 * (10 * n * n * c * c + 4 * n ** 3 * c + 2 * n * n * c * 4)
    trans = 24 * n * n * c * c
    single = 8 * n * cs * cs + 4 * n * n * cs + 6 * n * cs * 4 * cs + 2 * n * n * c * 16
    return tri + att + trans + single


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm = sorted(int(r[1]) for r in self.rows if len(r) >= 9 and r[1].isdigit())
        mx = [int(r[2]) for r in self.rows if len(r) >= 9 and r[2].isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) < 9:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], d.get("bf16_tflops_sustained", d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


def read_profile(lib, ctx, steps):
    """Per-kernel-class CUDA-event totals recorded by the library since the last read."""
    per_kernel = {}
    for k, name in enumerate(KERNEL_CLASSES):
        ms, cnt = C.c_float(), C.c_int()
        lib.xfold_profile_read(ctx, k, C.byref(ms), C.byref(cnt))
        if cnt.value:
            per_kernel[name] = {"ms_per_step": ms.value / steps, "launches_per_step": cnt.value // steps,
                                "avg_ms": ms.value / cnt.value}
    return per_kernel


# ---------------------------------------------------------------------------------------------------------------
# reference arm: the reference's CPU implementation of the path on the host cores
# ---------------------------------------------------------------------------------------------------------------
def cpu_block_ms(O, n, seed, threads, row_chunk=32, ref_block=None):
    """One Pairformer block in fp32 on `threads` host threads: ms.  ``ref_block``: the reference's own
    DistributePairformerBlock class (imported from a checkout); otherwise the oracle port."""
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(seed)
    st = O.make_pairformer_block_state(g, "")
    z, s, pm, sm = O.make_inputs(seed + 1, n, pad_frac=0.1)
    with torch.no_grad():
        if ref_block is not None:
            m = ref_block()
            m.load_state_dict(st)
            t0 = time.perf_counter()
            m(z, pm, s, sm.bool())
            return (time.perf_counter() - t0) * 1e3
        t0 = time.perf_counter()
        O.pairformer_block(st, "", z, pm, s, sm, row_chunk=row_chunk)
        return (time.perf_counter() - t0) * 1e3


def load_reference_block(ref_dir):
    """The reference's own block class, importable only where a checkout of the reference is mounted (its third-party
    base classes come from the stand-ins under oracle/).  Returns None when no checkout is given or found."""
    if not ref_dir or not os.path.isdir(os.path.join(ref_dir, "src", "distributed_xfold")):
        return None
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ref_standins
    ref_standins.install(os.path.join(ref_dir, "src"))
    from distributed_xfold.distribute_utils import DeviceMesh
    from distributed_xfold.nn.d_pairformer import DistributePairformerBlock
    mesh = DeviceMesh(1, dp_size=1, tp_size=1)
    return lambda: DistributePairformerBlock(mesh)


def cpu_sample_tokens(O, n_full, cores, budget_ms, calls, ref_block=None):
    """Largest token count (n_full, or n_full halved as often as needed) at which `calls` single-block runs fit the budget."""
    t256 = cpu_block_ms(O, 256, 11, cores, ref_block=ref_block)
    n_s = n_full
    while n_s > 256 and t256 * (n_s / 256) ** 3 * calls > budget_ms:
        n_s //= 2
    return n_s, t256


def run_reference(args):
    """`--impl reference`: the reference's CPU implementation of the path on all host cores.  Its fused LIBXSMM kernels
    cannot be built (the submodule is absent), so this is the reference's own Python forward when a checkout is given
    (--reference-dir, kind "reference-python"), else the fp32 oracle port.  A step is ONE block of the trunk at the
    largest token count that keeps the whole run within a few minutes, scaled to the 48-block recycle."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if args.workload == "trimul":
        from bench_multi import run_reference_trimul
        return run_reference_trimul(args)
    O = ge.load_oracle()
    cores = os.cpu_count() or 1
    ref_block = load_reference_block(args.reference_dir)
    kind = "reference-python" if ref_block is not None else "port"
    n_full, blocks = args.tokens, args.blocks
    warm = min(args.warmup, 1)
    n_s, _ = cpu_sample_tokens(O, n_full, cores, 200e3, args.steps + warm, ref_block)
    scale = flops_block(n_full) / flops_block(n_s)
    for _ in range(warm):
        cpu_block_ms(O, n_s, 12, cores, ref_block=ref_block)
    ts = [cpu_block_ms(O, n_s, 13 + i, cores, ref_block=ref_block) for i in range(args.steps)]
    ms_recycle = sum(ts) / len(ts) * scale * blocks
    sample = (f"each step = 1 of {blocks} blocks at N={n_s}, fp32, {cores} host threads, "
              + ("the reference's DistributePairformerBlock.forward" if ref_block is not None else "oracle port")
              + ("" if n_s == n_full else f", scaled to N={n_full} by the block's flop ratio {scale:.2f}")
              + f", x{blocks} blocks")
    cfg = workload_config(args, args.gpus)
    cfg["workload"] += f" [CPU arm: {sample}]"
    line = {"impl": "reference", "metric": "pairformer_ms_per_recycle", "value": ms_recycle, "unit": "ms",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": warm, "ms_per_step": ms_recycle,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": cfg,
            "cpu_baseline": {"value": ms_recycle, "unit": "ms", "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": ms_recycle, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def workload_config(args, world):
    if args.workload == "trimul":
        return {"workload": f"TriangleMultiplication outgoing + incoming, N={args.tokens} tokens, c_z=128, bf16, seed-1 "
                            "random-init weights (BASELINE config 2)",
                "tokens": args.tokens, "parallelism": f"pair rows over {world} GPU(s)",
                "l2": "inputs (151 MB pair representation at N=768) exceed the 126 MB L2; no flush between steps"}
    if args.workload == "diffusion":
        return {"workload": f"24-block DiffusionTransformer (c_token 768, 16 heads x 48), N={args.tokens} tokens, bf16, "
                            f"frozen synthetic trunk output, {world} sample(s), one per GPU, fixed per-sample noise "
                            "seeds (BASELINE config 5); a step = one denoising step of every sample",
                "tokens": args.tokens, "samples": world, "parallelism": f"samples over {world} GPU(s) (replicas)",
                "l2": "the bf16 pair logits read per step (3.2 GB at N=2048) exceed the 126 MB L2; no flush between steps"}
    return {"workload": f"48-block Pairformer trunk, one recycle, N={args.tokens} tokens, c_z=128, c_s=384, "
                        "bf16, seed-2 random-init weights, 10% padding mask (BASELINE config 3)",
            "tokens": args.tokens, "blocks": args.blocks, "parallelism": f"pair rows over {world} GPU(s)",
            "l2": "inputs (268 MB pair representation) exceed the 126 MB L2; no flush between steps"}


def roofline_entry(name, per_kernel, ms_step, n, tf_sust, hbm, which, traffic=None, traffic_note=None):
    c = 128
    alg = {  # algorithmic flops / bytes per launch at N tokens
        "trimul_contract": ("tensor", 2.0 * n ** 3 * c),
        "attention": ("tensor", 4.0 * n ** 3 * c),
        "trimul_proj": ("tensor", 2.0 * n * n * c * 5 * c),
        "linear": ("tensor", 2.0 * n * n * c * 4 * c),
        "linear_swiglu": ("tensor", 2.0 * n * n * c * 8 * c),
        "linear_gate_resid": ("hbm", 3.0 * n * n * c * 2),
        "layernorm": ("hbm", 2.0 * n * n * c * 2),
        "channel_ln": ("hbm", 2.0 * n * n * c * 2),
    }
    if name not in per_kernel or name not in alg:
        return None
    bound, work = alg[name]
    sec = per_kernel[name]["avg_ms"] * 1e-3
    if bound == "tensor":
        ach, pk, unit = work / sec / 1e12, tf_sust, "TFLOP/s"
    else:
        ach, pk, unit = work / sec / 1e9, hbm, "GB/s"
    return {"kernel": name, "bound": bound, "achieved": ach, "peak": pk, "unit": unit, "frac": ach / pk,
            "avg_launch_ms": per_kernel[name]["avg_ms"], "traffic": traffic, "traffic_unit": traffic_note,
            "peak_source": which + (" (sustained)" if bound == "tensor" else ""),
            "share_of_step": per_kernel[name]["ms_per_step"] / ms_step}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="trunk", choices=["trunk", "trimul", "diffusion"])
    ap.add_argument("--tokens", type=int, default=None)
    ap.add_argument("--blocks", type=int, default=48)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--reference-dir", default=os.environ.get("XFOLD_REFERENCE"),
                    help="checkout of the reference project; when given, the CPU arm drives its own Python forward")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 1)
    if args.tokens is None:
        args.tokens = {"trunk": 1024, "trimul": 768, "diffusion": 2048}[args.workload]
    if args.impl == "reference":
        return run_reference(args)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload == "trimul":
        from bench_multi import run_trimul
        return run_trimul(args, world, rank, local_rank)
    if args.workload == "diffusion":
        from bench_multi import run_diffusion
        return run_diffusion(args, world, rank, local_rank)
    if world > 1:
        from bench_multi import run_multi  # row-sharded path
        return run_multi(args, world, rank, local_rank)

    ge.load_package()
    from distributed_xfold_b200 import _cabi, ops
    O = ge.load_oracle()  # weight / input factory only (plus the CPU baseline leg below)
    torch.cuda.set_device(local_rank)
    dev = f"cuda:{local_rank}"
    n, nb = args.tokens, args.blocks
    lib, ctx = _cabi.load(), _cabi.ctx(local_rank)

    g = torch.Generator().manual_seed(2)
    blocks = []
    for i in range(nb):
        st = O.make_pairformer_block_state(g, "")
        blocks.append(ops.PackedPairformerBlock(st, "", dev))
        del st
    trunk = ops.PackedPairformerStack(blocks)
    z_h, s_h, pm_h, sm_h = O.make_inputs(3, n, pad_frac=0.1)
    z_h, s_h = z_h.to(torch.bfloat16).pin_memory(), s_h.to(torch.bfloat16).pin_memory()
    pm_h, sm_h = pm_h.pin_memory(), sm_h.pin_memory()
    z_out_h, s_out_h = torch.empty_like(z_h).pin_memory(), torch.empty_like(s_h).pin_memory()
    z0, s0 = z_h.to(dev), s_h.to(dev)
    pm, sm = pm_h.to(dev), sm_h.to(dev)
    z, s = torch.empty_like(z0), torch.empty_like(s0)

    def recycle():  # the product's trunk loop: one C-ABI call for all blocks
        ops.pairformer_stack_(z, s, pm, sm, trunk)

    def step_resident():
        z.copy_(z0)
        s.copy_(s0)
        recycle()

    def step_e2e():
        z.copy_(z_h, non_blocking=True)
        s.copy_(s_h, non_blocking=True)
        pm.copy_(pm_h, non_blocking=True)
        sm.copy_(sm_h, non_blocking=True)
        recycle()
        z_out_h.copy_(z, non_blocking=True)
        s_out_h.copy_(s, non_blocking=True)

    lib.xfold_profile_enable(ctx, 0)
    for _ in range(args.warmup):
        step_resident()
    ops.synchronize_and_check(local_rank)
    assert torch.isfinite(z.float()).all(), "non-finite pair representation after warm-up"

    # ---- timed region (device resident, instrumentation off), CUDA events on the launching stream ---------
    sampler = ClockSampler(local_rank)
    sampler.start()
    l0 = lib.xfold_launch_count(ctx)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        step_resident()
    e1.record()
    torch.cuda.synchronize()
    ms_step = e0.elapsed_time(e1) / args.steps
    launches = int(lib.xfold_launch_count(ctx) - l0)
    clocks = sampler.stop()
    ops.synchronize_and_check(local_rank)

    # ---- end to end with host buffers ---------------------------------------------------------
    step_e2e()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        step_e2e()
    e1.record()
    torch.cuda.synchronize()
    ms_e2e = e0.elapsed_time(e1) / args.steps
    h2d = z_h.numel() * 2 + s_h.numel() * 2 + pm_h.numel() * 4 + sm_h.numel() * 4
    d2h = z_h.numel() * 2 + s_h.numel() * 2
    ops.synchronize_and_check(local_rank)

    # ---- per-kernel table: a separate pass with every launch bracketed by events (not part of `value`) ----
    prof_steps = min(args.steps, 2)
    lib.xfold_profile_enable(ctx, 1)
    step_resident()  # fills the event pool
    torch.cuda.synchronize()
    read_profile(lib, ctx, 1)
    e0.record()
    for _ in range(prof_steps):
        step_resident()
    e1.record()
    torch.cuda.synchronize()
    ms_prof = e0.elapsed_time(e1) / prof_steps
    per_kernel = read_profile(lib, ctx, prof_steps)
    lib.xfold_profile_enable(ctx, 0)

    # ---- roofline of the dominant kernel + the TriMul contraction -----------------------------
    hbm, tf_burst, tf_sust, which = peaks()
    # DRAM bytes per launch (read + write; for attention dram__bytes.sum.per_second x duration) from the one-kernel ncu captures summarised
    # under profiles/, taken at N = 1024; these kernels' traffic grows with N^2, so other sizes are scaled by (N / 1024)^2
    ncu_traffic_n1024 = {"attention": 1.370e9, "trimul_contract": 0.537e9 + 0.235e9}
    tnote = "bytes per launch (ncu, one launch at N=1024" + ("" if n == 1024 else ", scaled by N^2") + ")"
    top = max(per_kernel, key=lambda k: per_kernel[k]["ms_per_step"]) if per_kernel else None

    def roof(name):
        tr = ncu_traffic_n1024.get(name)
        return roofline_entry(name, per_kernel, ms_prof, n, tf_sust, hbm, which,
                              None if tr is None else tr * (n / 1024.0) ** 2, tnote if tr is not None else None)

    line = {"metric": "pairformer_ms_per_recycle", "value": ms_step, "unit": "ms", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "ms_per_block": ms_step / nb, "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(args, 1), "clocks": clocks, "gpu_launches": launches,
            "e2e": {"value": ms_e2e, "unit": "ms", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "roofline": roof(top), "roofline_trimul_contract": roof("trimul_contract"),
            "model_tflops": flops_block(n) * nb / (ms_step * 1e-3) / 1e12,
            "kernels_note": f"per-kernel CUDA-event times from a separate instrumented pass ({ms_prof:.1f} ms per step)",
            "kernels": per_kernel}

    if not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        n_s, t256 = cpu_sample_tokens(O, n, cores, 30e3, 1)
        tb = cpu_block_ms(O, n_s, 13, cores) if n_s > 256 else t256
        scale = flops_block(n) / flops_block(n_s)
        line["cpu_baseline"] = {"value": tb * scale * nb, "unit": "ms", "cores": cores, "kind": "port",
                                "sample": f"one fp32 oracle block at N={n_s} on {cores} threads"
                                          + ("" if n_s == n else f", scaled by the block flop ratio {scale:.2f}")
                                          + f", x{nb} blocks"}
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
