#!/usr/bin/env python
"""NeuS2 training-step benchmark on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N=1): BASELINE config 1 -- static NeuS training on the seeded analytic sphere scene (64 RGBA views 512x512,
Fibonacci-sphere cameras, fov 40 deg), hash grid 16 levels x 2 features, T=2^19, SDF MLP 48->64->16, colour MLP
48->64->64->16, target batch 2^18 samples/step, 128^3 occupancy grid, eikonal weight 0.1, Adam lr 1e-2.  A step is one
call of the reference's Testbed::train(batch): occupancy update when due, ray sampling, fused forward, loss + compaction,
fused forward+backward, Adam(+EMA), batch re-tune.  Synthetic data, random-init (geometric-init) weights; the scene is
pre-trained for `--pretrain` untimed steps so the occupancy grid and the rays-per-batch tuner are in steady state.

`value` = training samples per second with everything resident in HBM (CUDA events on the library's stream, max over
ranks).  `e2e` = the same through the host-facing call with host buffers every step (camera block H2D from pinned memory,
counters + losses D2H, host sync).  `--impl reference` times the CPU oracle (OpenMP port of the same step) instead.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "neus_train_samples_per_s"
UNIT = "samples/s"
BATCH = 1 << 18


def workload_config(n_gpus):
    return {"workload": "BASELINE config 1: sphere scene 64x512x512 RGBA, hash grid L16 F2 T2^19, batch 2^18 samples/step, "
                        "eikonal 0.1, Adam lr 1e-2", "global_batch": BATCH * n_gpus, "n_views": 64, "resolution": 512,
            "parallelism": "dp%d (rays sharded, one gradient all-reduce per step)" % n_gpus if n_gpus > 1 else "single GPU",
            "l2": "per-step working set (~0.6 GB: 25 MB grid + 25 MB gradients + 200 MB Adam state + sample buffers) exceeds the "
                  "126 MB L2, no explicit flush"}


class ClockSampler:
    """nvidia-smi clocks / throttle reasons during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.lines, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for nme, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nme)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def occupancy_updates_between(step0, n_steps):
    """How many of the steps [step0, step0+n) run training_prep_nerf (src/testbed.cu:2659)."""
    c = 0
    for s in range(step0, step0 + n_steps):
        skip = min(max(s // 16, 1), 16)
        c += (s % skip == 0)
    return c


def make_scene(device):
    from neus2_b200 import synthetic as S
    return S.render_sphere_views(64, 512, 512, fov_deg=40.0, radius=0.3, seed=0, device=device)


def cuda_view(ptr, nbytes):
    """uint8 torch tensor over a raw device pointer (memory owned by libneus2b.so)."""
    import torch

    class _V:
        pass
    v = _V()
    v.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}
    return torch.as_tensor(v, device="cuda")


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from neus2_b200 import _lib as L
    from neus2_b200 import ops
    from neus2_b200 import synthetic as S
    from neus2_b200.testbed import Testbed

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback of the product path)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    L.lib()

    scene = make_scene("cuda")
    kw = {"learning_rate": args.lr} if args.lr else {}
    if args.forward_windows is not None:
        kw["forward_windows"] = [int(v) for v in args.forward_windows.split(",") if v]
    tb = Testbed(batch_size=BATCH, world_size=world, rank=rank, **kw)
    px = scene["pixels"].cpu().numpy()
    cams = [scene[k].cpu().numpy() for k in ("xforms", "focal", "principal")]
    tb.load_training_data(px, *cams)
    ng = L.grid_n_params(tb.config.grid)
    tb.set_params(S.init_params(ng, seed=1337))
    ptrs = tb.device_ptrs()
    stream = torch.cuda.ExternalStream(ptrs["stream"])
    from neus2_b200.parallel import DataParallelTrainer
    dp = DataParallelTrainer(tb, ng)

    def step(read_stats=False, next_cameras=None):
        return dp.step(read_stats=read_stats, next_cameras=next_cameras)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.pretrain):
        step()
    st = step(read_stats=True)
    for _ in range(max(args.warmup - 1, 0)):
        step()
    # ---- device-resident timing
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    first_step = args.pretrain + max(args.warmup, 1)
    # The cost of a step drifts with the training state (the surface sharpens, fewer samples per ray survive compaction, more
    # rays are drawn), so the K device-resident steps and the K end-to-end steps are interleaved in blocks: both arms see
    # the same mix of states.  Device-resident block: steps enqueued back to back, timed with CUDA events on the training
    # stream.  End-to-end block: the host-facing call with the camera block uploaded from pinned host memory and the step's
    # statistics read back (host sync) every step.
    n_blocks = min(4, args.steps)
    sizes = [args.steps // n_blocks + (1 if b < args.steps % n_blocks else 0) for b in range(n_blocks)]
    ms = ms_e2e = 0.0
    kernel_ms_sum, kernel_launches = 0.0, 0
    launches_before = L.launch_count()
    step_first = int(st.training_step) + max(args.warmup - 1, 0)
    for nb in sizes:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for _ in range(nb):
            step()
        e1.record(stream)
        barrier()
        ms += e0.elapsed_time(e1)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        tb.profile_train_kernel(nb)  # CUDA-event pairs around the fused forward+backward launch of these steps
        t0.record(stream)
        # one camera upload and one statistics read-back per step; the camera block of the NEXT step is uploaded behind this
        # step's backward pass, so that the samples drawn ahead (during the gradient exchange on several GPUs, during the
        # host's wait for the statistics on one) already use it
        tb.update_cameras(*cams)
        for _ in range(nb):
            st = step(read_stats=True, next_cameras=cams)
        t1.record(stream)
        barrier()
        ms_e2e += t0.elapsed_time(t1)
        a, b = tb.profile_train_kernel(0)
        kernel_ms_sum, kernel_launches = kernel_ms_sum + a, kernel_launches + b
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms, ms_e2e], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = t.tolist()
    ms_step = ms / args.steps
    value = BATCH * world * args.steps / (ms * 1e-3)
    e2e_value = BATCH * world * args.steps / (ms_e2e * 1e-3)
    # kernels of libneus2b.so launched inside the two timed arms (counted by the library at every launch site); NCCL's
    # all-reduce kernels on several GPUs are not the library's and are not counted
    launches = L.launch_count() - launches_before

    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16 (fp32 accumulate)",
            "data": "synthetic", "config": workload_config(world),
            "gpu_launches_note": "libneus2b.so kernels inside both timed arms (2 x steps training steps)",
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": int(sum(c.nbytes for c in cams)), "d2h_bytes_per_step": 32},
            "gpu_launches": launches, "clocks": clocks,
            "train_state": {"timed_steps": [step_first, int(st.training_step)], "training_step": int(st.training_step),
                            "rays_per_batch": int(st.rays_per_batch),
                            "samples_before_compaction": int(st.measured_batch_size_before_compaction), "samples_evaluated": int(st.n_samples_evaluated),
                            "samples_after_compaction": int(st.measured_batch_size), "loss": float(st.loss),
                            "ek_loss": float(st.ek_loss), "overflow": int(st.overflow)}}

    # ---- where the gradient exchange sits in a step (several GPUs): CUDA events over 20 more training steps, outside `value`
    if world > 1:
        ex = dp.probe_exchange(20)
        t = torch.tensor([ex["allreduce_ms"], ex["allreduce_with_generation_beside_ms"]], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        line["exchange"] = dict(zip(("allreduce_ms", "allreduce_with_generation_beside_ms"), [round(v, 4) for v in t.tolist()]),
                                note="max over ranks of per-rank medians, on the training stream; 25 MB fp16 grid gradient + 48 KB fp32 MLP/variance "
                                     "gradient per step; the next step's samples are drawn on a second stream beside the exchange and the optimizer pass")

    # ---- mesh extraction at 512^3, sharded by z-slab over the ranks (SDF lattice with the EMA weights, marching cubes with
    # global numbering, counters all-gathered, slices gathered into rank 0): not part of `value`
    if not args.no_mesh:
        line["mesh_512"] = mesh_record(tb, rank, world, args.mesh_res)
    if rank == 0:
        # ---- roofline of the dominant kernel (fused forward+backward over the 2^18 compacted samples), timed alone
        line["roofline"] = roofline_train_kernel(tb, ptrs, st, ng, kernel_ms_sum / max(kernel_launches, 1), kernel_launches)
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(tb, sample=args.cpu_sample)
        print(json.dumps(line), flush=True)
    barrier()
    tb.close()
    if world > 1:
        dist.destroy_process_group()


def mesh_record(tb, rank, world, res):
    """Times the sharded extraction (max over ranks, CUDA events) and checks on rank 0 that it equals this GPU's own
    extraction of the whole lattice."""
    import hashlib
    import torch
    import torch.distributed as dist

    def run():
        return tb.compute_marching_cubes_mesh_sharded_device(res, rank, world, use_ema=True)
    run()  # warm-up (allocations, NCCL point-to-point connections)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    v, i = run()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    rec = {"res": res, "ms": float(ms.item()), "n_gpus": world, "sharding": "z-slab per rank, global numbering on the devices"}
    if rank == 0:
        def digest(a, b):
            return hashlib.sha1(a.contiguous().cpu().numpy().tobytes() + b.contiguous().cpu().numpy().tobytes()).hexdigest()[:16]
        rec.update(verts=int(v.shape[0]), triangles=int(i.shape[0] // 3), sha1=digest(v, i))
        if world > 1:
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            v1, i1 = tb.compute_marching_cubes_mesh(res, use_ema=True)
            t1.record()
            torch.cuda.synchronize()
            rec.update(single_gpu_ms=t0.elapsed_time(t1), equal_to_single_gpu=bool(digest(v1, i1.view(torch.int32)) == rec["sha1"]))
    return rec


# Figures of one launch of the fused forward+backward kernel at 2^18 samples from the `ncu --set full` capture summarised
# in profiles/neus_tc_kernel_train_2p18_samples.txt (constants copied from that capture, not measured by this run):
# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum: the hash table and its gradient table stay in L2, what
# reaches HBM is their first touch plus the sample streams), L2 sectors requested by the SMs, tensor-pipe activity.
TRAIN_KERNEL_DRAM_BYTES = 59966464 + 516096
TRAIN_KERNEL_L2_SECTORS = 26909409
TRAIN_KERNEL_TENSOR_PIPE_PCT = 5.4


def roofline_train_kernel(tb, ptrs, st, ng, ms_in_step, launches_in_step):
    """Roofline line of the dominant kernel (fused forward+backward, 2^18 compacted samples per launch).
    `achieved` uses the kernel's average duration inside the timed steps (CUDA-event pairs on the training stream around
    each launch).  The same kernel is also timed alone on a 2^18-sample batch drawn around the trained surface with the
    L2 flushed before every launch (`ms_per_launch_cold_l2`).  Algorithmic bytes per sample: 28 (coordinate) + 32
    (output gradient) + 512 (one gather pass over 16 levels x 8 corners x 4 B) + 512 (one merged scatter pass) = 1084 B."""
    import torch
    from neus2_b200 import ops
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak, src, tensor_peak = 6650.0, "fallback", 1400.0
    if os.path.exists(peaks_path):
        try:
            pk = json.load(open(peaks_path))
            peak, src = float(pk["hbm_gbs"]), "measured"
            tensor_peak = float(pk.get("bf16_tflops_sustained", tensor_peak))  # the kernel is timed inside a long step
        except (KeyError, ValueError, OSError):
            pass
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    n = BATCH
    # samples in a shell around the r=0.3 sphere, ordered along rays like a real batch (consecutive samples 1.7e-3 apart)
    rays = n // 64
    o = torch.randn(rays, 3, device="cuda", generator=g)
    o = 0.5 + 0.3 * o / o.norm(dim=1, keepdim=True)
    d = torch.randn(rays, 3, device="cuda", generator=g)
    d = d / d.norm(dim=1, keepdim=True)
    t = (torch.arange(64, device="cuda") - 32) * (math.sqrt(3) / 1024)
    pos = (o[:, None, :] + t[None, :, None] * d[:, None, :]).reshape(-1, 3).clamp(0.0, 1.0)
    coords = torch.zeros(n, 7, device="cuda")
    coords[:, :3] = pos
    coords[:, 4:] = ((d + 1) * 0.5)[:, None, :].expand(rays, 64, 3).reshape(-1, 3)
    dl = (torch.randn(n, 16, device="cuda", generator=g) * 1e-2).half()
    params = cuda_view(ptrs["params"], (12288 + ng + 4) * 2).view(torch.float16)
    gm = torch.zeros(12288, device="cuda")
    gg = torch.zeros(ng, dtype=torch.float16, device="cuda")
    gv = torch.zeros(4, device="cuda")
    desc = tb.config.grid
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    times = []
    for it in range(8):
        flush.zero_()  # write a buffer larger than L2 between timed launches
        torch.cuda.synchronize()
        e0.record()
        ops.neus_train(desc, params, coords, dl, n, gm, gg, gv)
        e1.record()
        torch.cuda.synchronize()
        if it >= 3:
            times.append(e0.elapsed_time(e1))
    ms_cold = sum(times) / len(times)
    ms = ms_in_step if launches_in_step else ms_cold
    bytes_per_sample = 28 + 32 + 512 + 512
    achieved = bytes_per_sample * n / (ms * 1e-3) / 1e9
    return {"kernel": "neus_tc_kernel<TRAIN> (tcgen05 fused forward+backward, 2^18 samples per launch)", "bound": "hbm",
            "achieved": achieved, "peak": peak,
            "peak_source": src + " (MEASURED_PEAKS.json hbm_gbs)" if src == "measured" else "fallback 6.65 TB/s",
            "unit": "GB/s", "frac": achieved / peak, "traffic": TRAIN_KERNEL_DRAM_BYTES,
            "traffic_source": "constant from the ncu capture summarised in profiles/neus_tc_kernel_train_2p18_samples.txt",
            "bound_note": "the denominator is the HBM copy peak, but the kernel is not HBM-bound: its algorithmic bytes are table "
                          "gathers and reductions served by L1/L2 (DRAM traffic is 0.2x the algorithmic bytes); what limits it is the "
                          "latency of those gathers and reductions at 16 resident warps per SM and the per-sample arithmetic around them",
            "l2_sector_gbs": TRAIN_KERNEL_L2_SECTORS * 32 / (ms * 1e-3) / 1e9,
            "tensor_pipe_active_pct_ncu": TRAIN_KERNEL_TENSOR_PIPE_PCT,
            "tensor_frac": 96256 * n / (ms * 1e-3) / 1e12 / tensor_peak,
            "tensor_peak_tflops": tensor_peak, "ms_per_launch": ms,
            "launches_timed": launches_in_step, "ms_per_launch_cold_l2": ms_cold,
            "algorithmic_bytes_per_sample": bytes_per_sample, "flop_per_sample": 96256,
            "achieved_tflops": 96256 * n / (ms * 1e-3) / 1e12}


def run_kernel_only(args):
    """Small stand-alone case of one fused kernel for profiler captures:
    `ncu ... python bench.py --kernel train --kernel-n 131072 --kernel-iters 3`."""
    import numpy as np
    import torch
    from neus2_b200 import _lib as L
    from neus2_b200 import ops
    from neus2_b200 import synthetic as S
    torch.cuda.set_device(0)
    desc = L.grid_desc()
    ng = L.grid_n_params(desc)
    if args.kernel == "adam":
        n = 12288 + ng + 4
        f32 = lambda: torch.randn(n, device="cuda") * 1e-3
        master, m, v, ema = f32(), f32(), f32().abs(), f32()
        P = torch.zeros(n, dtype=torch.float16, device="cuda")
        Pe = torch.zeros(n, dtype=torch.float16, device="cuda")
        gm, gv = torch.randn(12288, device="cuda"), torch.zeros(4, device="cuda")
        gsrc = (torch.randn(ng, device="cuda") * (torch.rand(ng, device="cuda") < 0.3)).half()
        gg = gsrc.clone()
        cfg = L.AdamCfg(1e-2, 0.9, 0.99, 1e-15, 1e-6, 0.95, 128.0, 10, 12288)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        times = []
        for it in range(args.kernel_iters):
            gg.copy_(gsrc)
            flush.zero_()
            torch.cuda.synchronize()
            e0.record()
            ops.adam_step(cfg, gm, gg, gv, master, m, v, P, Pe, ema)
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        print(json.dumps({"kernel": "adam", "n_params": n, "ms": times, "GBps": 40.0 * n / (min(times) * 1e-3) / 1e9}))
        return
    if args.kernel == "mesh":
        # BASELINE config 4's mesh half: SDF on a res^3 lattice through the fused SDF kernel, then marching cubes
        import time
        from neus2_b200.testbed import Testbed
        res = args.mesh_res
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if world > 1:
            import torch.distributed as dist
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
            dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))))
        tb = Testbed(batch_size=1 << 18)
        tb.set_params(S.init_params(ng, seed=1337))  # geometric initialisation: a sphere-like SDF
        if world > 1:
            # sharded by z-slab: every rank evaluates its layers and runs marching cubes on them, the parts are gathered
            # (pickled host arrays over the process group) and merged on the host; time = the slowest rank
            rank = int(os.environ.get("RANK", "0"))
            out = []
            for it in range(args.kernel_iters):
                dist.barrier()
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                v, i = tb.compute_marching_cubes_mesh_sharded(res, rank, world, use_ema=False)
                t = torch.tensor([time.perf_counter() - t0], device="cuda")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                out.append({"wall_s": float(t.item()), "verts": int(len(v)), "triangles": int(len(i)) // 3})
            if rank == 0:
                print(json.dumps({"kernel": "mesh", "res": res, "n_gpus": world, "sharded_by": "z-slab", "runs": out}))
            tb.close()
            dist.destroy_process_group()
            return
        e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        stream = torch.cuda.ExternalStream(tb.device_ptrs()["stream"])
        out = []
        for it in range(args.kernel_iters):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            e[0].record(stream)
            sdf = tb.sdf_grid(res, use_ema=False)
            e[1].record(stream)
            stream.synchronize()
            e[2].record()
            v, i = ops.marching_cubes(sdf)
            e[3].record()
            torch.cuda.synchronize()
            out.append({"sdf_ms": e[0].elapsed_time(e[1]), "mc_ms": e[2].elapsed_time(e[3]), "wall_s": time.perf_counter() - t0,
                        "verts": int(v.shape[0]), "triangles": int(i.shape[0]) // 3})
            del sdf, v, i
        print(json.dumps({"kernel": "mesh", "res": res, "runs": out}))
        tb.close()
        return
    if args.kernel == "config2":
        # BASELINE config 2 stand-in: torus + rounded box, 49 views at 1600x1200, batch 2^19, progressive levels (8 + 2 per 500
        # steps); device time per step over --steps steps after --pretrain steps, then the mesh against the analytic surface
        from neus2_b200.testbed import Testbed
        scene = S.render_csg_views(49, 1600, 1200, device="cuda", seed=0)
        tb = Testbed(batch_size=1 << 19, progressive_start_levels=8, progressive_levels_per_increment=2, progressive_steps_per_increment=500,
                     **({"learning_rate": args.lr} if args.lr else {}))
        tb.load_training_data(scene["pixels"].cpu().numpy(), *[scene[k].cpu().numpy() for k in ("xforms", "focal", "principal")])
        del scene
        tb.set_params(S.init_params(ng, seed=1337))
        stream = torch.cuda.ExternalStream(tb.device_ptrs()["stream"])
        runs = []
        for block in range(args.kernel_iters):
            tb.train(args.pretrain, read_stats=False)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            tb.train(args.steps, read_stats=False)
            e1.record(stream)
            st = tb.train(1)
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / args.steps
            runs.append({"training_step": int(st.training_step), "ms_per_step": ms, "samples_per_s": (1 << 19) / (ms * 1e-3),
                         "rays_per_batch": int(st.rays_per_batch), "samples_before_compaction": int(st.measured_batch_size_before_compaction),
                         "samples_after_compaction": int(st.measured_batch_size), "loss": float(st.loss), "ek_loss": float(st.ek_loss),
                         "overflow": int(st.overflow)})
        v, i = tb.compute_marching_cubes_mesh(256)
        err = S.csg_sdf(v).abs()
        seen = v[:, 2] > 0.5  # the cameras sit on a cap above the object: its underside is never observed
        print(json.dumps({"kernel": "config2", "runs": runs, "mesh": {"res": 256, "verts": int(v.shape[0]), "triangles": int(i.shape[0]) // 3,
                                                                        "mean_abs_sdf": float(err.mean()), "p99_abs_sdf": float(err.quantile(0.99)),
                                                                        "upper_half_mean_abs_sdf": float(err[seen].mean()),
                                                                        "upper_half_p99_abs_sdf": float(err[seen].quantile(0.99))}}))
        tb.close()
        return
    if args.kernel == "config3":
        # BASELINE config 3 stand-in: a sequence of --frames frames of the config-1 sphere under a seeded per-frame rigid motion
        # (rotation <= 5 deg, translation <= 0.02 per frame) and a sinusoidal radial bulge of amplitude 0.03, 24 views at 512 x 512
        # per frame; 2 000 steps on the first frame, then --frame-steps steps per later frame (the first quarter of them on the
        # learned rigid motion alone), warm-started from the previous frame.  Reports wall-clock per frame: image upload, frame
        # switch and training (the frames are rendered ahead, which is data preparation).
        import time
        from neus2_b200.testbed import Testbed
        n_frames, per_frame = args.frames, args.frame_steps
        poses = S.sequence_poses(n_frames, seed=0)
        tb = Testbed(batch_size=1 << 18, predict_global_movement=1, predict_global_movement_training_step=max(per_frame // 4, 1),
                     finetune_global_movement=1, reset_density_grid_after_global_movement=0, after_learning_rate=1e-3, ek_loss_weight=0.01,
                     base_training_step=100, valid_level_scale=0.02, base_valid_level_scale=0.2)

        def views(f):
            sc = S.render_sphere_views(24, 512, 512, device="cuda", seed=0, rotation=poses[f][0], translation=poses[f][1], radius=poses[f][2])
            return [sc[k].cpu().numpy() for k in ("pixels", "xforms", "focal", "principal")]
        t0 = time.perf_counter()
        tb.load_training_data(*views(0))
        tb.set_params(S.init_params(ng, seed=1337))
        st = tb.train(args.first_frame_steps)
        torch.cuda.synchronize()
        first_s = time.perf_counter() - t0
        per, losses = [], []
        for f in range(1, n_frames):
            data = views(f)  # (rendered outside the timed part)
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            tb.next_frame(*data)
            st = tb.train(per_frame)
            torch.cuda.synchronize()
            per.append(time.perf_counter() - t1)
            losses.append(float(st.loss))
        per_sorted = sorted(per)
        frame, R_acc, t_acc, _ = tb.movement()
        print(json.dumps({"kernel": "config3", "frames": n_frames, "views": 24, "resolution": 512, "first_frame_steps": args.first_frame_steps,
                          "steps_per_later_frame": per_frame, "first_frame_s": first_s,
                          "later_frame_ms": {"median": 1e3 * per_sorted[len(per) // 2], "mean": 1e3 * sum(per) / len(per),
                                             "p90": 1e3 * per_sorted[int(0.9 * (len(per) - 1))], "max": 1e3 * per_sorted[-1]},
                          "ms_per_step_in_later_frames": 1e3 * sum(per) / len(per) / per_frame,
                          "final_loss": losses[-1], "max_loss": max(losses), "frame": frame,
                          "accumulated_rotation_deg": float(np.degrees(np.arcsin(min(1.0, float(np.linalg.norm(R_acc - R_acc.T)) / (2.0 * 2.0 ** 0.5))))),
                          "accumulated_translation": [float(v) for v in t_acc]}))
        tb.close()
        return
    if args.kernel == "render":
        # one frame of Testbed.render (1 sample per pixel) of the briefly trained config-1 scene, host image out
        import time
        from neus2_b200.testbed import Testbed
        scene = S.render_sphere_views(64, 512, 512, device="cuda", seed=0)
        tb = Testbed(batch_size=1 << 18, **({"learning_rate": args.lr} if args.lr else {}))
        tb.load_training_data(scene["pixels"].cpu().numpy(), *[scene[k].cpu().numpy() for k in ("xforms", "focal", "principal")])
        tb.set_params(S.init_params(ng, seed=1337))
        tb.train(args.pretrain)
        X = scene["xforms"][7].cpu().numpy()
        tb.camera_matrix = np.stack([X[0:3], X[3:6], X[6:9], X[9:12]], 1)
        tb.fov = args.render_fov
        tb.background_color = [0.0, 0.0, 0.0, 0.0]
        w, h = args.render_res
        out = []
        for it in range(args.kernel_iters):
            t0 = time.perf_counter()
            img = tb.render(w, h, spp=1, linear=False)
            out.append({"wall_ms": (time.perf_counter() - t0) * 1e3, "device_ms": tb.last_render_device_ms,
                        "samples": tb.last_render_samples, "coverage": float((img[..., 3] > 0.5).mean())})
        print(json.dumps({"kernel": "render", "width": w, "height": h, "runs": out}))
        tb.close()
        return
    p = S.init_params(ng, seed=1337)
    rng = np.random.default_rng(9)
    p[12288:12288 + ng] = rng.uniform(-1e-2, 1e-2, ng)
    p[:3072].reshape(64, 48)[:, 3:35] = rng.normal(0, 0.05, (64, 32))
    params = torch.from_numpy(p).cuda().half()
    n = args.kernel_n
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    rays = max(n // 64, 1)
    o = torch.randn(rays, 3, device="cuda", generator=g)
    o = 0.5 + 0.3 * o / o.norm(dim=1, keepdim=True)
    d = torch.randn(rays, 3, device="cuda", generator=g)
    d = d / d.norm(dim=1, keepdim=True)
    t = (torch.arange(64, device="cuda") - 32) * (math.sqrt(3) / 1024)
    pos = (o[:, None, :] + t[None, :, None] * d[:, None, :]).reshape(-1, 3).clamp(0.0, 1.0)[:n]
    n = pos.shape[0]
    coords = torch.zeros(n, 7, device="cuda")
    coords[:, :3] = pos
    coords[:, 4:] = ((d + 1) * 0.5)[:, None, :].expand(rays, 64, 3).reshape(-1, 3)[:n]
    dl = (torch.randn(n, 16, device="cuda", generator=g) * 1e-2).half()
    gm = torch.zeros(12288, device="cuda")
    gg = torch.zeros(ng, dtype=torch.float16, device="cuda")
    gv = torch.zeros(4, device="cuda")
    out = torch.zeros(n, 16, dtype=torch.float16, device="cuda")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for it in range(args.kernel_iters):
        torch.cuda.synchronize()
        e0.record()
        if args.kernel == "train":
            ops.neus_train(desc, params, coords, dl, n, gm, gg, gv)
        else:
            ops.neus_forward(desc, params, coords, out=out)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    print(json.dumps({"kernel": args.kernel, "n": n, "ms": times}))


def cpu_baseline(tb, sample=1 << 18):
    """The CPU oracle (OpenMP port of the same step) on a bounded sample of the workload: fused forward on 2x sample
    pre-compaction samples, forward+backward on `sample` compacted samples, Adam over all parameters; scaled to
    samples/s.  Reported beside the GPU number, not a target."""
    import numpy as np
    from oracle import oracle as O
    cores = os.cpu_count() or 1
    O.set_num_threads(cores)
    d = O.grid_desc()
    p32 = tb.get_params()
    params = O.f16_bits(p32)
    rng = np.random.default_rng(3)
    n = sample
    dirs = rng.normal(size=(n, 3))
    dirs /= np.linalg.norm(dirs, axis=1, keepdims=True)
    coords = np.zeros((n, 7), np.float32)
    coords[:, :3] = np.clip(0.5 + dirs * (0.3 + rng.normal(0, 0.02, (n, 1))), 0, 1)
    coords[:, 4:] = rng.random((n, 3))
    g = O.f16_bits(rng.normal(0, 1e-2, (n, 16)))
    m, v = np.zeros_like(p32), np.zeros_like(p32)
    pe, em = np.zeros(p32.size, np.uint16), p32.copy()
    cfg = O.AdamCfg(1e-2, 0.9, 0.99, 1e-15, 1e-6, 0.95, 128.0, 1, 12288)
    pre = np.concatenate([coords, coords])
    reps, t0 = 0, time.time()
    while reps < 16 and (reps == 0 or time.time() - t0 < 10.0):  # about 10 s of CPU work
        O.neus_forward(d, params, pre)                                      # pre-compaction pass (N_pre ~ 2 N)
        grad = O.neus_backward(d, params, coords, g, indeed_batch_size=n)  # forward + backward on the compacted batch
        O.adam_step(cfg, grad.astype(np.float32), p32, m, v, params, pe, em)
        reps += 1
    dt = time.time() - t0
    return {"value": n * reps / dt, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": "%d steps of %d compacted samples (+2x pre-compaction forward, Adam over all 12.6 M parameters), %.1f s"
                      % (reps, n, dt)}


def run_reference(args):
    """Reference arm: the reference has no CPU path and its CUDA build needs the un-vendored tiny-cuda-nn fork, so the
    timed thing is the CPU oracle (OpenMP port of the same step) on all host cores, on a bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    import numpy as np
    from oracle import oracle as O
    from neus2_b200 import synthetic as S
    cores = os.cpu_count() or 1
    O.set_num_threads(cores)  # torchrun pins OMP_NUM_THREADS=1: the reference arm uses every host core
    d = O.grid_desc()
    ng = O.grid_n_params(d)
    p32 = S.init_params(ng, seed=1337)
    params = O.f16_bits(p32)
    rng = np.random.default_rng(3)

    def make_batch(n):
        dirs = rng.normal(size=(n, 3))
        dirs /= np.linalg.norm(dirs, axis=1, keepdims=True)
        c = np.zeros((n, 7), np.float32)
        c[:, :3] = np.clip(0.5 + dirs * (0.3 + rng.normal(0, 0.02, (n, 1))), 0, 1)
        c[:, 4:] = rng.random((n, 3))
        return c, O.f16_bits(rng.normal(0, 1e-2, (n, 16)))

    m, v = np.zeros_like(p32), np.zeros_like(p32)
    pe, em = np.zeros(p32.size, np.uint16), p32.copy()
    # size the per-step sample so that the K + W steps end within ~2.5 minutes
    coords, g = make_batch(2048)
    t0 = time.time()
    O.neus_forward(d, params, np.concatenate([coords, coords]))
    O.neus_backward(d, params, coords, g, indeed_batch_size=2048)
    rate = 2048 / max(time.time() - t0, 1e-3)
    n = int(min(max(rate * 150.0 / (args.steps + args.warmup), 512), min(args.cpu_sample * 4, BATCH))) // 128 * 128
    coords, g = make_batch(n)

    t_fb = t_adam = 0.0

    def step(k, timed):
        nonlocal t_fb, t_adam
        a = time.time()
        O.neus_forward(d, params, np.concatenate([coords, coords]))
        grad = O.neus_backward(d, params, coords, g, indeed_batch_size=n)
        b = time.time()
        cfg = O.AdamCfg(1e-2, 0.9, 0.99, 1e-15, 1e-6, 0.95, 128.0, k + 1, 12288)
        O.adam_step(cfg, grad.astype(np.float32), p32, m, v, params, pe, em)
        if timed:
            t_fb += b - a
            t_adam += time.time() - b

    for k in range(args.warmup):
        step(k, False)
    for k in range(args.steps):
        step(args.warmup + k, True)
    # a full step = the sample part scaled to 2^18 samples + the optimizer pass, which always covers every parameter
    dt = t_fb * (BATCH / n) + t_adam
    value = BATCH * args.steps / dt
    sample = ("%d compacted samples per step (+2x pre-compaction forward) scaled to the 2^18-sample step, "
              "plus Adam over all 12.6 M parameters every step" % n)
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp16 storage, fp32 math (CPU)", "data": "synthetic",
            "config": workload_config(world),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "the reference's own CUDA build needs the un-vendored tiny-cuda-nn fork (empty submodule) and it has "
                    "no CPU path: this arm times the CPU oracle port"}
    loop = reference_loop_on_gpu()
    if loop is not None:
        line["reference_loop_on_gpu"] = loop
    print(json.dumps(line), flush=True)


def reference_loop_on_gpu():
    """Beside the CPU figure: the reference's own headless training loop (its unmodified sources compiled over this repository's
    tiny-cuda-nn headers, oracle/_ref/libref_testbed.so) on the same workload on this GPU: the reference's host code, ray-march, loss
    and occupancy kernels and its NerfNetwork / Trainer objects, with this repository's layered kernels under them.  It is not the
    reference's tiny-cuda-nn build, which cannot be produced.  Runs as a child process; None when there is no GPU or no such library."""
    import subprocess
    import torch
    here = os.path.dirname(os.path.abspath(__file__))
    if not torch.cuda.is_available() or not os.path.exists(os.path.join(here, "oracle", "_ref", "libref_testbed.so")):
        return None
    try:
        r = subprocess.run([sys.executable, os.path.join(here, "oracle", "run_ref_testbed.py"), "--views", "64", "--res", "512", "--batch", str(BATCH),
                            "--warmup", "520", "--steps", "200"], capture_output=True, text=True, timeout=600, cwd=here)
        out = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    except Exception as e:  # the measurement is an extra: never fail the arm over it
        return {"unavailable": "%s: %s" % (type(e).__name__, str(e)[:200])}
    if "ms_per_step" in out:
        out["value"] = BATCH / (out["ms_per_step"] * 1e-3)
        out["unit"] = UNIT
        out["what"] = ("the reference's unmodified headless Testbed loop over this repository's tiny-cuda-nn headers (layered kernels), "
                       "steps 520-720 of config 1, wall clock around 200 frame() calls")
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--pretrain", type=int, default=500)
    ap.add_argument("--lr", type=float, default=0.0, help="override the Adam learning rate of BASELINE config 1 (1e-2), e.g. to time late training states")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--forward-windows", default=None, help="cumulative window ends of the step's network pass, e.g. 16,64 ('' = every sample like the reference; default: the library's)")
    ap.add_argument("--cpu-sample", type=int, default=1 << 18)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--kernel", default=None, choices=["train", "forward", "adam", "mesh", "render", "config2", "config3"], help="run one fused kernel alone (profiling)")
    ap.add_argument("--kernel-n", type=int, default=1 << 17)
    ap.add_argument("--kernel-iters", type=int, default=3)
    ap.add_argument("--frames", type=int, default=100, help="--kernel config3: frames of the sequence")
    ap.add_argument("--frame-steps", type=int, default=100, help="--kernel config3: training steps per frame after the first")
    ap.add_argument("--first-frame-steps", type=int, default=2000)
    ap.add_argument("--mesh-res", type=int, default=512)
    ap.add_argument("--no-mesh", action="store_true", help="skip the 512^3 mesh extraction record behind the timed steps")
    ap.add_argument("--render-res", type=int, nargs=2, default=[1600, 1200], help="width height of --kernel render (DTU images are 1600x1200)")
    ap.add_argument("--render-fov", type=float, default=30.0)
    args = ap.parse_args()
    if args.kernel:
        run_kernel_only(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
