"""Multi-GPU leg of bench.py (launched by torchrun, one rank per GPU): the same 48-block Pairformer
recycle with the pair representation partitioned by token rows over the ranks (strong scaling)."""
from __future__ import annotations

import ctypes as C
import json
import os

import torch
import torch.distributed as dist

import __graft_entry__ as ge


def run_multi(args, world, rank, local_rank):
    from bench import KERNEL_CLASSES, ClockSampler, flops_block, peaks, workload_config
    ge.load_package()
    from distributed_xfold_b200 import _cabi, ops, row_sharded
    O = ge.load_oracle()  # weight / input factory only
    torch.cuda.set_device(local_rank)
    dev = f"cuda:{local_rank}"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=torch.device(dev))
    n, nb = args.tokens, args.blocks
    lib, ctx = _cabi.load(), _cabi.ctx(local_rank)

    g = torch.Generator().manual_seed(2)
    packed = []
    for _ in range(nb):
        st = O.make_pairformer_block_state(g, "")
        packed.append(ops.PackedPairformerBlock(st, "", dev))
        del st
    z_h, s_h, pm_h, sm_h = O.make_inputs(3, n, pad_frac=0.1)
    sh = row_sharded.RowSharding(n)
    stages = row_sharded.CudaStages()
    if os.environ.get("XFOLD_CHANNEL_SHARDED") in ("0", "1"):
        sh.force_channel_sharded = os.environ["XFOLD_CHANNEL_SHARDED"] == "1"
    peer = sh.enable_peer_exchange(dev) and os.environ.get("XFOLD_NO_PEER") != "1"
    if not peer:
        sh.peer = None
    z_h = z_h[sh.rows].to(torch.bfloat16).contiguous().pin_memory()
    s_h = s_h.to(torch.bfloat16).pin_memory()
    z_out_h, s_out_h = torch.empty_like(z_h).pin_memory(), torch.empty_like(s_h).pin_memory()
    z0, s0 = z_h.to(dev), s_h.to(dev)
    pm, sm = pm_h.to(dev), sm_h.to(dev)
    pmt = pm.t().contiguous()
    state = {"z": torch.empty_like(z0), "s": torch.empty_like(s0)}

    def recycle():
        z, s = state["z"], state["s"]
        for w in packed:
            z, s = row_sharded.pairformer_block(sh, stages, z, s, pm, pmt, sm, w)
        state["z"], state["s"] = z, s

    def step_resident():
        state["z"] = z0.clone()
        state["s"] = s0.clone()
        recycle()

    def step_e2e():
        state["z"] = z_h.to(dev, non_blocking=True)
        state["s"] = s_h.to(dev, non_blocking=True)
        recycle()
        z_out_h.copy_(state["z"], non_blocking=True)
        s_out_h.copy_(state["s"], non_blocking=True)

    def timed(fn, steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(args.warmup):
        step_resident()
    ops.synchronize_and_check(local_rank)
    assert torch.isfinite(state["z"].float()).all()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    lib.xfold_profile_enable(ctx, 1)
    l0 = lib.xfold_launch_count(ctx)
    ms_step = timed(step_resident, args.steps)
    launches = int(lib.xfold_launch_count(ctx) - l0)
    clocks = sampler.stop() if rank == 0 else None
    per_kernel = {}
    for k, name in enumerate(KERNEL_CLASSES):
        ms, cnt = C.c_float(), C.c_int()
        lib.xfold_profile_read(ctx, k, C.byref(ms), C.byref(cnt))
        if cnt.value:
            per_kernel[name] = {"ms_per_step": ms.value / args.steps, "launches_per_step": cnt.value // args.steps,
                                "avg_ms": ms.value / cnt.value}
    lib.xfold_profile_enable(ctx, 0)
    ops.synchronize_and_check(local_rank)

    step_e2e()
    ms_e2e = timed(step_e2e, args.steps)
    ops.synchronize_and_check(local_rank)
    lt = torch.tensor([launches], device=dev, dtype=torch.int64)
    dist.all_reduce(lt)

    if rank == 0:
        hbm, tf_burst, tf_sust, which = peaks()
        r = sh.r
        roof = None
        if "trimul_contract" in per_kernel:
            sec = per_kernel["trimul_contract"]["avg_ms"] * 1e-3
            ach = 2.0 * r * n * n * 128 / sec / 1e12
            roof = {"kernel": "trimul_contract", "bound": "tensor", "achieved": ach, "peak": tf_sust, "unit": "TFLOP/s",
                    "frac": ach / tf_sust, "traffic": None, "peak_source": which + " (sustained)",
                    "share_of_step": per_kernel["trimul_contract"]["ms_per_step"] / ms_step,
                    "note": "per-rank kernel: this rank's rows against all gathered rows of b"}
        kern_ms = sum(v["ms_per_step"] for v in per_kernel.values())
        line = {"metric": "pairformer_ms_per_recycle", "value": ms_step, "unit": "ms", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "ms_per_block": ms_step / nb,
                "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": workload_config(args, world), "clocks": clocks, "gpu_launches": int(lt.item()),
                "e2e": {"value": ms_e2e, "unit": "ms", "h2d_bytes_per_step": (z_h.numel() + s_h.numel()) * 2 * world,
                        "d2h_bytes_per_step": (z_h.numel() + s_h.numel()) * 2 * world},
                "roofline": roof, "model_tflops": flops_block(n) * nb / (ms_step * 1e-3) / 1e12,
                "rank0_kernel_ms_per_step": kern_ms, "rank0_exchange_and_glue_ms_per_step": ms_step - kern_ms, "peer_memory_transpose": bool(peer),
                "trimul_exchange": "channel slices (rows -> channels, product, rows back)" if sh.channel_sharded else "all-gather of b",
                "kernels": per_kernel}
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()
