"""Legs of bench.py beyond the single-GPU trunk recycle:

  run_multi             the 48-block Pairformer recycle with the pair representation partitioned by token rows over
                        the ranks (launched by torchrun, one rank per GPU; strong scaling), with a parity check of the
                        sharded block against the one-GPU block in the same run;
  run_trimul            BASELINE config 2: TriangleMultiplication outgoing + incoming at N = 768 on P GPUs;
  run_reference_trimul  the same on the host cores: P gloo ranks of the row-sharded TriangleMultiplication in fp32;
  run_diffusion         BASELINE config 5: the 24-block DiffusionTransformer at N = 2048, one sample per GPU.
"""
from __future__ import annotations

import json
import os
import sys
import time

import torch
import torch.distributed as dist

import __graft_entry__ as ge

NVLINK_GBS = 770.0  # measured peer-copy bandwidth per direction per GPU on this pool (nominal 900)


def _init(local_rank, world):
    torch.cuda.set_device(local_rank)
    dev = f"cuda:{local_rank}"
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(dev))
    return dev


def _timed(fn, steps, dev, world):
    """CUDA events on the launching stream, a barrier + synchronize on both sides, max over ranks."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def exchange_bytes_per_block(sh) -> float:
    """Bytes this rank sends over NVLink per Pairformer block: two distributed transposes, per TriangleMultiplication the
    other ranks' share of a, b and of the output rows (channel slices), and its rows of the two pair biases and of the
    pair logits to every other rank."""
    n, p, r = sh.n, sh.world, sh.r
    ld = (n + 7) // 8 * 8
    away = (p - 1) / p
    transposes = 2 * away * r * n * 128 * 2
    trimul = 2 * away * (2 * r * 128 * ld * 2 + (128 // p) * n * ld * 2)
    bias = (p - 1) * (4 + 4 + 16) * r * ld * 2
    return transposes + trimul + bias


def run_multi(args, world, rank, local_rank):
    from bench import ClockSampler, flops_block, peaks, read_profile, workload_config
    ge.load_package()
    from distributed_xfold_b200 import _cabi, ops, row_sharded
    O = ge.load_oracle()  # weight / input factory only
    dev = _init(local_rank, world)
    n, nb = args.tokens, args.blocks
    lib, ctx = _cabi.load(), _cabi.ctx(local_rank)

    g = torch.Generator().manual_seed(2)
    packed = []
    for _ in range(nb):
        st = O.make_pairformer_block_state(g, "")
        packed.append(ops.PackedPairformerBlock(st, "", dev))
        del st
    z_full_h, s_h, pm_h, sm_h = O.make_inputs(3, n, pad_frac=0.1)
    sh = row_sharded.RowSharding(n)
    trunk = row_sharded.ShardedTrunk(sh, dev)  # peer-mapped buffers + the library's shard context
    stack = ops.PackedPairformerStack(packed)
    z_h = z_full_h[sh.rows].to(torch.bfloat16).contiguous().pin_memory()
    s_h = s_h.to(torch.bfloat16).pin_memory()
    z_out_h, s_out_h = torch.empty_like(z_h).pin_memory(), torch.empty_like(s_h).pin_memory()
    z0, s0 = z_h.to(dev), s_h.to(dev)
    pm, sm = pm_h.to(dev), sm_h.to(dev)
    s_dev = torch.empty_like(s0)

    # ---- parity of the sharded path against the one-GPU path, in this very run -------------------------------
    # Every rank runs the first block on its row shard; rank 0 also runs it on the whole pair representation through
    # the one-GPU entry point and compares (relative Frobenius over unpadded positions).
    trunk.load(z0)
    ss = s0.clone()
    zs = trunk.run(ss, pm, sm, ops.PackedPairformerStack(packed[:1]))
    z_sharded = sh.gather_rows(zs.contiguous())
    ops.synchronize_and_check(local_rank)
    parity = None
    if rank == 0:
        z1 = z_full_h.to(torch.bfloat16).to(dev)
        s1 = s0.clone()
        ops.pairformer_block_(z1, s1, pm, sm, packed[0])
        ops.synchronize_and_check(local_rank)
        valid = pm > 0

        def relf(a, b):
            return float((a.double() - b.double()).norm() / b.double().norm())
        parity = {"z": relf(z_sharded.float()[valid], z1.float()[valid]), "s": relf(ss.float()[sm > 0], s1.float()[sm > 0]),
                  "what": "relative Frobenius error of block 1 on the row shards (gathered) against the one-GPU block, unpadded positions"}
        assert parity["z"] <= 2e-2 and parity["s"] <= 2e-2, parity
        del z1, s1
    del z_sharded, zs, ss, z_full_h
    torch.cuda.empty_cache()

    def step_resident():  # one C-ABI call per rank runs all blocks, exchanges included
        trunk.load(z0)
        s_dev.copy_(s0)
        trunk.run(s_dev, pm, sm, stack)

    def step_e2e():
        trunk.shard_view().copy_(z_h, non_blocking=True)
        s_dev.copy_(s_h, non_blocking=True)
        out = trunk.run(s_dev, pm, sm, stack)
        z_out_h.copy_(out, non_blocking=True)
        s_out_h.copy_(s_dev, non_blocking=True)

    lib.xfold_profile_enable(ctx, 0)
    for _ in range(args.warmup):
        step_resident()
    ops.synchronize_and_check(local_rank)
    assert torch.isfinite(trunk.shard_view().float()).all()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    l0 = lib.xfold_launch_count(ctx)
    ms_step = _timed(step_resident, args.steps, dev, world)
    launches = int(lib.xfold_launch_count(ctx) - l0)
    clocks = sampler.stop() if rank == 0 else None
    ops.synchronize_and_check(local_rank)

    step_e2e()
    ms_e2e = _timed(step_e2e, args.steps, dev, world)
    ops.synchronize_and_check(local_rank)

    # per-kernel table: a separate pass with every launch bracketed by events (not part of `value`)
    prof_steps = min(args.steps, 2)
    lib.xfold_profile_enable(ctx, 1)
    step_resident()
    torch.cuda.synchronize()
    read_profile(lib, ctx, 1)
    ms_prof = _timed(step_resident, prof_steps, dev, world)
    per_kernel = read_profile(lib, ctx, prof_steps)
    lib.xfold_profile_enable(ctx, 0)
    lt = torch.tensor([launches], device=dev, dtype=torch.int64)
    dist.all_reduce(lt)

    if rank == 0:
        hbm, tf_burst, tf_sust, which = peaks()
        r = sh.r
        roof = None
        if "trimul_contract" in per_kernel:
            sec = per_kernel["trimul_contract"]["avg_ms"] * 1e-3
            # a rank contracts 128 / world channels of N x N x N, in as many launches as the stage is chunked into
            per_launch = 2.0 * nb * (2.0 * n ** 3 * 128 / world) / per_kernel["trimul_contract"]["launches_per_step"]
            ach = per_launch / sec / 1e12
            roof = {"kernel": "trimul_contract", "bound": "tensor", "achieved": ach, "peak": tf_sust, "unit": "TFLOP/s",
                    "frac": ach / tf_sust, "traffic": None, "peak_source": which + " (sustained)",
                    "share_of_step": per_kernel["trimul_contract"]["ms_per_step"] / ms_prof,
                    "note": "per-rank launches (this rank's channels, one chunk of them per launch); no ncu capture is "
                            "taken of a multi-rank run, so traffic is not reported here"}
        xbytes = exchange_bytes_per_block(sh) * nb
        xms = per_kernel.get("peer_exchange", {}).get("ms_per_step")
        exchange = {"bytes_sent_per_rank_per_step": xbytes, "nvlink_floor_ms": xbytes / (NVLINK_GBS * 1e9) * 1e3,
                    "peer_exchange_kernels_ms": xms, "nvlink_peak_gbs": NVLINK_GBS,
                    "frac_of_nvlink": None if not xms else xbytes / (xms * 1e-3) / 1e9 / NVLINK_GBS,
                    "form": "channel slices (rows -> channels, product, rows back), incoming product on the same planes"}
        kern_ms = sum(v["ms_per_step"] for v in per_kernel.values())
        line = {"metric": "pairformer_ms_per_recycle", "value": ms_step, "unit": "ms", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "ms_per_block": ms_step / nb,
                "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": workload_config(args, world), "clocks": clocks, "gpu_launches": int(lt.item()),
                "e2e": {"value": ms_e2e, "unit": "ms", "h2d_bytes_per_step": (z_h.numel() + s_h.numel()) * 2 * world,
                        "d2h_bytes_per_step": (z_h.numel() + s_h.numel()) * 2 * world},
                "parity_vs_1gpu": parity, "roofline": roof, "exchange": exchange,
                "model_tflops": flops_block(n) * nb / (ms_step * 1e-3) / 1e12,
                "kernels_note": f"per-kernel CUDA-event times of rank 0 from a separate instrumented pass ({ms_prof:.1f} ms per step)",
                "rank0_kernel_ms_per_step": kern_ms, "rank0_glue_ms_per_step": ms_prof - kern_ms,
                "peer_memory_exchange": True, "kernels": per_kernel}
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------------------------
# BASELINE config 2: TriangleMultiplication outgoing + incoming, N = 768, pair rows over P ranks
# ---------------------------------------------------------------------------------------------------------------
def _trimul_flops(n, c=128):
    return 2 * (2.0 * n ** 3 * c + 12.0 * n * n * c * c)


def run_trimul(args, world, rank, local_rank):
    from bench import ClockSampler, peaks, read_profile, workload_config
    ge.load_package()
    from distributed_xfold_b200 import _cabi, ops, row_sharded
    O = ge.load_oracle()
    dev = _init(local_rank, world)
    n = args.tokens
    lib, ctx = _cabi.load(), _cabi.ctx(local_rank)
    g = torch.Generator().manual_seed(1)
    st = {}
    st.update(O.make_trimul_state(g, "out."))
    st.update(O.make_trimul_state(g, "in."))
    w_out, w_in = ops.PackedTriMul(st, "out.", dev), ops.PackedTriMul(st, "in.", dev)
    z_full, _, pm_h, _ = O.make_inputs(4, n, pad_frac=0.0)
    sh = row_sharded.RowSharding(n) if world > 1 else None
    rows = sh.rows if sh is not None else slice(0, n)
    z_h = z_full[rows].to(torch.bfloat16).contiguous().pin_memory()
    out_h = torch.empty_like(z_h).pin_memory()
    z0 = z_h.to(dev)
    pm = pm_h.to(dev)
    pmt = pm.t().contiguous()
    state = {"z": torch.empty_like(z0)}
    if sh is not None:
        sh.enable_peer_exchange(dev)
        stages = row_sharded.CudaStages()

    def op():
        if sh is None:
            ops.triangle_multiplication_(state["z"], pm, w_out, True)
            ops.triangle_multiplication_(state["z"], pm, w_in, False)
        else:
            state["z"] = row_sharded.trimul_out_in(sh, stages, state["z"], pm, pmt, w_out, w_in)

    def step_resident():
        state["z"] = z0.clone()
        op()

    def step_e2e():
        state["z"] = z_h.to(dev, non_blocking=True)
        op()
        out_h.copy_(state["z"], non_blocking=True)

    # parity against the CPU oracle on a sub-problem is the tests' job; here: sharded against one GPU, same run
    parity = None
    if sh is not None:
        step_resident()
        zsh = sh.gather_rows(state["z"].contiguous())
        if rank == 0:
            z1 = z_full.to(torch.bfloat16).to(dev)
            ops.triangle_multiplication_(z1, pm, w_out, True)
            ops.triangle_multiplication_(z1, pm, w_in, False)
            parity = {"z": float((zsh.double() - z1.double()).norm() / z1.double().norm())}
            assert parity["z"] <= 2e-2, parity
            del z1
        del zsh
    for _ in range(args.warmup):
        step_resident()
    ops.synchronize_and_check(local_rank)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    l0 = lib.xfold_launch_count(ctx)
    ms = _timed(step_resident, args.steps, dev, world)
    launches = int(lib.xfold_launch_count(ctx) - l0)
    clocks = sampler.stop() if rank == 0 else None
    step_e2e()
    ms_e2e = _timed(step_e2e, args.steps, dev, world)
    lib.xfold_profile_enable(ctx, 1)
    step_resident()
    torch.cuda.synchronize()
    read_profile(lib, ctx, 1)
    ms_prof = _timed(step_resident, 2, dev, world)
    per_kernel = read_profile(lib, ctx, 2)
    lib.xfold_profile_enable(ctx, 0)
    ops.synchronize_and_check(local_rank)
    lt = torch.tensor([launches], device=dev, dtype=torch.int64)
    if world > 1:
        dist.all_reduce(lt)
    if rank == 0:
        hbm, tf_burst, tf_sust, which = peaks()
        fl = _trimul_flops(n)
        ach = fl / (ms * 1e-3) / 1e12 / world  # per GPU
        roof = {"kernel": "TriangleMultiplication out + in (all launches of the op)", "bound": "tensor", "achieved": ach,
                "peak": tf_sust, "unit": "TFLOP/s per GPU", "frac": ach / tf_sust, "traffic": None,
                "peak_source": which + " (sustained)"}
        if "trimul_contract" in per_kernel:
            sec = per_kernel["trimul_contract"]["avg_ms"] * 1e-3
            a2 = 2.0 * n ** 3 * 128 / world / sec / 1e12
            roof["contraction_kernel"] = {"achieved": a2, "frac": a2 / tf_sust, "avg_launch_ms": sec * 1e3}
        line = {"metric": "trimul_out_in_ms", "value": ms, "unit": "ms", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(args, world),
                "clocks": clocks, "gpu_launches": int(lt.item()),
                "e2e": {"value": ms_e2e, "unit": "ms", "h2d_bytes_per_step": z_h.numel() * 2 * world,
                        "d2h_bytes_per_step": z_h.numel() * 2 * world},
                "parity_vs_1gpu": parity, "roofline": roof, "kernels": per_kernel}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _gloo_trimul_rank(rank, world, port, n, threads, steps, ref_dir, ret):
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import __graft_entry__ as ge_
    O = ge_.load_oracle()
    torch.set_num_threads(threads)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(1)
    st = {}
    st.update(O.make_trimul_state(g, "out."))
    st.update(O.make_trimul_state(g, "in."))
    z, _, pm, _ = O.make_inputs(4, n, pad_frac=0.0)
    info = O.ShardInfo(n, world)
    sl = info.slices[rank]

    def gather_dim(dim):  # all-gather of b over the sharded axis (nn/d_triangle_multiplication.py:74-79), ragged sizes padded
        def gather(t):
            if world == 1:
                return t
            pad = max(info.sizes)
            buf = t.new_zeros(t.shape[:dim] + (pad,) + t.shape[dim + 1:])
            buf.narrow(dim, 0, t.shape[dim]).copy_(t)
            parts = [torch.empty_like(buf) for _ in range(world)]
            dist.all_gather(parts, buf)
            return torch.cat([p.narrow(dim, 0, sz) for p, sz in zip(parts, info.sizes)], dim)
        return gather

    times = []
    with torch.no_grad():
        for it in range(steps + 1):
            dist.barrier()
            t0 = time.perf_counter()
            # outgoing takes the row shard, incoming the column shard (nn/d_triangle_multiplication.py:48-99)
            o = O.triangle_multiplication_sharded(st, "out.", z[sl], pm[sl], gather_dim(1), True)
            i = O.triangle_multiplication_sharded(st, "in.", z[:, sl], pm[:, sl], gather_dim(2), False)
            dist.barrier()
            if it:
                times.append((time.perf_counter() - t0) * 1e3)
            del o, i
    if rank == 0:
        ret["ms"] = sum(times) / len(times)
    dist.destroy_process_group()


def run_reference_trimul(args):
    """BASELINE config 2 on the host: the row-sharded TriangleMultiplication (outgoing on the row shard, incoming on the
    column shard, all-gather of b over gloo) in fp32, P ranks x (cores / P) threads; the oracle's restatement of
    nn/d_triangle_multiplication.py:48-99."""
    import torch.multiprocessing as mp
    from bench import workload_config
    ge.load_package()
    from distributed_xfold_b200.distribute_utils import find_free_port
    cores = os.cpu_count() or 1
    p = max(args.gpus, 1)
    threads = max(cores // p, 1)
    n_full = args.tokens
    n_s = n_full
    # ~3 s per direction at N = 768 on 8 threads: bound the sample so that steps + 1 passes stay within a few minutes
    while n_s > 192 and 6.0 * (n_s / 768) ** 3 * (8 / max(cores, 1)) * (args.steps + 1) > 150:
        n_s //= 2
    ret = mp.Manager().dict()
    mp.spawn(_gloo_trimul_rank, args=(p, find_free_port(), n_s, threads, args.steps, args.reference_dir, ret), nprocs=p,
             join=True)
    scale = _trimul_flops(n_full) / _trimul_flops(n_s)
    ms = ret["ms"] * scale
    sample = (f"TriangleMultiplication out + in at N={n_s}, fp32 oracle port, {p} gloo rank(s) x {threads} threads"
              + ("" if n_s == n_full else f", scaled to N={n_full} by the flop ratio {scale:.2f}"))
    cfg = workload_config(args, p)
    cfg["workload"] += f" [CPU arm: {sample}]"
    line = {"impl": "reference", "metric": "trimul_out_in_ms", "value": ms, "unit": "ms", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": 1, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg,
            "cpu_baseline": {"value": ms, "unit": "ms", "cores": p * threads, "kind": "port", "sample": sample},
            "e2e": {"value": ms, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------
# BASELINE config 5: diffusion samples data-parallel over the GPUs (replicas; one gather at the end)
# ---------------------------------------------------------------------------------------------------------------
def run_diffusion(args, world, rank, local_rank):
    from bench import ClockSampler, peaks, read_profile, workload_config
    ge.load_package()
    from distributed_xfold_b200 import _cabi, diffusion, ops
    O = ge.load_oracle()
    dev = _init(local_rank, world)
    n = args.tokens
    lib, ctx = _cabi.load(), _cabi.ctx(local_rank)
    g = torch.Generator().manual_seed(7)
    st = O.make_diffusion_transformer_state(g, "")
    tr = diffusion.PackedDiffusionTransformer(st, "", dev)
    del st
    # frozen synthetic trunk output (replicated conditioning), per-sample noise from a fixed per-sample seed
    gz = torch.Generator().manual_seed(8)
    pair_cond = torch.randn(n, n, 128, generator=gz, dtype=torch.float32).to(torch.bfloat16).to(dev)
    single_cond = torch.randn(n, 384, generator=gz).to(torch.bfloat16).to(dev)
    mask = torch.ones(n, device=dev)
    my_samples = diffusion.shard_samples(world, world, rank)           # ShardInfo rule: one sample per rank here
    acts_h = torch.stack([torch.randn(n, 768, generator=torch.Generator().manual_seed(1000 + i)).to(torch.bfloat16)
                          for i in range(my_samples.start, my_samples.stop)]).pin_memory()
    out_h = torch.empty_like(acts_h).pin_memory()
    act0 = acts_h.to(dev)
    logits = tr.pair_logits(pair_cond)                                  # once per inference (step-invariant)
    del pair_cond
    ops.synchronize_and_check(local_rank)
    state = {"a": act0.clone()}

    def step_resident():
        tr.forward(state["a"], mask, single_cond, logits)

    def step_e2e():
        state["a"].copy_(acts_h, non_blocking=True)
        tr.forward(state["a"], mask, single_cond, logits)
        out_h.copy_(state["a"], non_blocking=True)

    for _ in range(args.warmup):
        step_resident()
    ops.synchronize_and_check(local_rank)
    assert torch.isfinite(state["a"].float()).all()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    l0 = lib.xfold_launch_count(ctx)
    ms = _timed(step_resident, args.steps, dev, world)
    launches = int(lib.xfold_launch_count(ctx) - l0)
    clocks = sampler.stop() if rank == 0 else None
    step_e2e()
    ms_e2e = _timed(step_e2e, args.steps, dev, world)
    # the one collective of the path: the samples' results gathered on every rank (d_alphafold3.py:460-472)
    gathered = None
    if world > 1:
        gathered = torch.empty((world,) + tuple(state["a"].shape[1:]), dtype=state["a"].dtype, device=dev)
        dist.all_gather_into_tensor(gathered, state["a"].contiguous())
        assert torch.isfinite(gathered.float()).all()
    lib.xfold_profile_enable(ctx, 1)
    step_resident()
    torch.cuda.synchronize()
    read_profile(lib, ctx, 1)
    _timed(step_resident, 2, dev, world)
    per_kernel = read_profile(lib, ctx, 2)
    lib.xfold_profile_enable(ctx, 0)
    ops.synchronize_and_check(local_rank)
    lt = torch.tensor([launches], device=dev, dtype=torch.int64)
    if world > 1:
        dist.all_reduce(lt)
    if rank == 0:
        hbm, tf_burst, tf_sust, which = peaks()
        top = max(per_kernel, key=lambda k: per_kernel[k]["ms_per_step"])
        # flops of one denoising step of one sample: per block 4 projections (8 N c^2), attention (4 N^2 c),
        # AdaLN-Zero output (2 N c^2), transition (2 N c 4c + 2 N 2c c) and the conditioning GEMMs
        c, cc = 768, 384
        fl = 24 * (8.0 * n * c * c + 4.0 * n * n * c + 2.0 * n * c * c + 12.0 * n * c * c + 2 * (4.0 * n * cc * c) + 2 * (2.0 * n * cc * c))
        line = {"metric": "diffusion_sample_steps_per_s", "value": world * 1e3 / ms, "unit": "sample-steps/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": workload_config(args, world), "clocks": clocks, "gpu_launches": int(lt.item()),
                "e2e": {"value": world * 1e3 / ms_e2e, "unit": "sample-steps/s",
                        "h2d_bytes_per_step": acts_h.numel() * 2 * world, "d2h_bytes_per_step": acts_h.numel() * 2 * world},
                "roofline": {"kernel": top, "bound": "tensor", "achieved": fl / (ms * 1e-3) / 1e12, "peak": tf_sust,
                             "unit": "TFLOP/s per GPU (whole step)", "frac": fl / (ms * 1e-3) / 1e12 / tf_sust,
                             "traffic": None, "peak_source": which + " (sustained)"},
                "pair_logits_once_per_inference": True, "kernels": per_kernel}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
