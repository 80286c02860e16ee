"""Benchmark of the rasterizer hot path: frames/s of the forward render.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

Workload (default): benchmark configuration 1 - 3,000,000 Gaussians (64-component mixture, SH degree 3),
1297x840, HYBRID_BLEND K=16, 200 orbit cameras - as seeded synthetic data (htgs_b200/scenes.py).
One step = `--views-per-step` frames per GPU; with N GPUs the views are partitioned round-robin over
the ranks (weak scaling, no data-path collective).  The scene stays resident in HBM like model weights;
a frame's inputs are its camera matrices, its outputs the image and the depth map.

Prints ONE JSON line (rank 0).  `value` = frames/s with cameras resident on the device and outputs left
there; `e2e` = frames/s through the public Python surface (`rasterize`) with the camera copied from pinned
host memory and image + depth copied back to pinned host memory inside the timed region.
`--impl reference` runs the unmodified reference extension (built under baseline/_ref) through its own
`rasterize` on the same workload; if that extension or a GPU is missing it times the float64 CPU port of
the reference's forward (oracle/) on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

from htgs_b200 import parallel, scenes  # noqa: E402

KERNELS_PER_FRAME_NOTE = "preprocess, scan, emit, 3 per sort pass, ranges, blend"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--views-per-step", type=int, default=24)
    ap.add_argument("--driver", default="auto", choices=["auto", "async", "threads"],
                    help="how this library's arm keeps two frames in flight: async = ONE host thread queueing frames on two CUDA streams without "
                         "waiting (deferred status checks); threads = two host threads with blocking calls; auto = async")
    ap.add_argument("--train-steps", type=int, default=0, help="steps of the training leg appended to the default workload (0 = --steps)")
    ap.add_argument("--no-train-leg", action="store_true", help="default workload: skip the configuration-2 training leg")
    ap.add_argument("--streams", type=int, default=0,
                    help="frames in flight per GPU on this library's arm (host threads, one CUDA stream each); 0 = 2 if the host has at least 3 hardware threads per rank, else 1")
    ap.add_argument("--n-gaussians", type=int, default=3_000_000, help="scale the workload down for quick checks (invalid as a benchmark)")
    ap.add_argument("--blend-mode", type=int, default=0, choices=[0, 1, 2, 3], help="0 HYBRID_BLEND (the benchmark), 1 FIRST_K, 2 GLOBAL_ORDERING, 3 OIT: for profiling the other modes' kernels")
    ap.add_argument("--k", type=int, default=16, choices=[1, 2, 4, 8, 16, 32], help="K of HYBRID_BLEND / FIRST_K (16 is the benchmark)")
    ap.add_argument("--workload", default="render", choices=["render", "render_fast", "train"],
                    help="render: configuration 1 (default, the headline metric); train: configuration 2 (fwd+bwd, L1 loss, one view per GPU, gradient all-reduce)")
    ap.add_argument("--exchange", default="compact", choices=["rows", "compact", "compact-nccl", "overlap", "dense"],
                    help="train at N > 1: compact = every rank publishes 64 bytes per Gaussian its view kept and expands every rank's buffer into the "
                         "dense sums, reading the peers' buffers over NVLink inside the kernel (default; compact-nccl: through one all-gather instead); rows = the gradient rows of Gaussians some rank kept, summed after the backward; "
                         "overlap = the chain rule (optionally the whole backward pass) runs in ranges of Gaussians and each finished range's rows are summed "
                         "while the next is computed; dense = the dense tensors, after the backward")
    ap.add_argument("--exchange-single-rank", action="store_true", help="train at N = 1 with --exchange compact: run the exchange's machinery anyway (its local cost; what the ncu summaries of its kernels use)")
    ap.add_argument("--exchange-one-pass", action="store_true", help="--exchange compact with one or two ranks: form the sums the way more than two ranks do (local copies, one pass)")
    ap.add_argument("--exchange-chunks", type=int, default=4, help="ranges of Gaussians the backward pass is split into for --exchange overlap")
    ap.add_argument("--exchange-split-pass", action="store_true", help="--exchange overlap: split the per-tile pass along the ranges too (default: only the per-Gaussian chain rule)")
    ap.add_argument("--reference-kind", default="auto", choices=["auto", "cuda", "cpu"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-sample-views", type=int, default=12)
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.device_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        inside = [l for (t, l) in self.lines if t0 - 0.05 <= t <= t1 + 0.15] or [l for (_, l) in self.lines]
        for line in inside:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": float(max(mx)) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def load_measured_peaks():
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d.get("hbm_gbs", 6650.0)), "measured"
    return 6650.0, "fallback"


MODE_NAMES = ["HYBRID_BLEND", "ALPHA_BLEND_FIRST_K", "ALPHA_BLEND_GLOBAL_ORDERING", "OIT_BLEND"]


def make_workload(args):
    scene = scenes.outdoor_scene(n=args.n_gaussians, n_views=200, mode=args.blend_mode, K=args.k)
    headline = args.n_gaussians == 3_000_000 and args.blend_mode == 0 and args.k == 16
    name = "config1: 3M Gaussians SH3, 1297x840, HYBRID_BLEND K=16, 200 orbit views" if headline else \
        f"VARIANT of config1 ({args.n_gaussians} Gaussians, {MODE_NAMES[args.blend_mode]} K={args.k}) - not the benchmark number"
    return scene, name


def cpu_port_fps(scene, n_views: int):
    """float64 CPU port of the reference forward on all host cores, on a bounded sample of views."""
    from oracle import oracle
    oracle.build()
    cores = oracle.hardware_threads()
    idx = [int(i) for i in np.linspace(0, len(scene.views) - 1, n_views).astype(int)]
    t0 = time.time()
    for i in idx:
        oracle.render(scene, scene.views[i], mode=scene.mode, K=scene.K, dtype=np.float64, n_threads=cores)
    dt = time.time() - t0
    return len(idx) / dt, cores, f"{len(idx)} of {len(scene.views)} views (indices {idx}), whole forward per view, {dt:.1f} s"


def run_reference_cpu(args, scene, workload_name, rank, world):
    if rank != 0:
        return
    fps_list = []
    sample = ""
    cores = 0
    for _ in range(max(1, min(args.steps, 2))):
        fps, cores, sample = cpu_port_fps(scene, max(1, min(args.cpu_sample_views, 3)))
        fps_list.append(fps)
    fps = float(np.mean(fps_list))
    line = {"impl": "reference", "reference_kind": "cpu-port (float64 restatement of the reference forward; the reference has no CPU path)",
            "metric": "frames/s", "value": fps, "unit": "frames/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1000.0 * args.views_per_step / fps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64",
            "data": "synthetic", "config": {"workload": workload_name, "views_per_step_per_gpu": args.views_per_step},
            "cpu_baseline": {"value": fps, "unit": "frames/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": fps, "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def run_training(args, mod, is_reference, scene, tensors, cams_dev, settings, device, dist, rank, world, workload_name, steps=None, warmup=None):
    """Configuration 2: one view per GPU per step, forward + backward through `diff_rasterize` with an L1 loss against a
    seeded uniform target, gradients of the six rasterizer inputs all-reduced over the ranks (NCCL)."""
    import torch
    steps = args.steps if steps is None else steps
    warmup = args.warmup if warmup is None else warmup
    n_views = len(scene.views)
    v0 = scene.views[0]
    gen = torch.Generator(device="cpu").manual_seed(1234)
    target = torch.rand((3, v0.height, v0.width), generator=gen).to(device)
    # The model's parameters are raw (log-scales, unnormalised quaternions, opacity logits; Model.py:45-49 of the reference)
    # and activated inside autograd every step: element-wise PyTorch operations on the reference arm, as its model does,
    # the fused activation kernel (`htgs_activate`) on this library's arm.
    positions, scales, rotations, opacities, sh_0, sh_rest = tensors
    raw = [positions.clone(), scales.log(), rotations * 1.5, torch.special.logit(opacities.clamp(1e-6, 1.0 - 1e-6)), sh_0.clone(), sh_rest.clone()]
    leaves = [t.contiguous().requires_grad_(True) for t in raw]
    empty = torch.empty(0, device=device)
    if is_reference:
        def activate(raw_scales, raw_rotations, raw_opacities):
            return torch.exp(raw_scales), torch.nn.functional.normalize(raw_rotations), torch.special.expit(raw_opacities)
    else:
        from htgs_b200 import glue
        activate = glue.activate

    # Exchange: this library's arm sums only the gradient rows of Gaussians some rank's view kept (the others are zero on
    # every rank); the reference has no multi-GPU path and no such list, its arm all-reduces the dense tensors.
    sparse = not is_reference and ((dist is not None and args.exchange in ("rows", "overlap", "compact", "compact-nccl")) or
                                   (dist is None and args.exchange_single_rank and args.exchange in ("compact", "compact-nccl")))
    overlap = sparse and args.exchange == "overlap"
    compact = sparse and args.exchange in ("compact", "compact-nccl")
    xchg = None
    if sparse:
        from htgs_b200.torch_bindings import rasterization
        rasterization.track_training_visibility(True)
    if overlap:
        xchg = parallel.BackwardExchange(n_chunks=args.exchange_chunks, measure=True, split_pass=args.exchange_split_pass)
        rasterization.set_backward_hook(xchg)
    if compact:
        xchg = parallel.CompactExchange(transport="peer" if args.exchange == "compact" else "nccl")
        xchg.always_stage = bool(args.exchange_one_pass)
        compact_transport = xchg.prepare(scene.n, device)      # falls back to the all-gather transport on all ranks if the buffers cannot be mapped
        rasterization.set_backward_hook(xchg)
    exchanged_rows = []
    gathered_bytes = []

    def step(s):
        vi = (s + rank * (n_views // world)) % n_views      # the views of a step are spread evenly over the orbit, as a random batch would be
        for l in leaves:
            l.grad = None
        act_scales, act_rotations, act_opacities = activate(leaves[1], leaves[2], leaves[3])
        image = mod.diff_rasterize(leaves[0], act_scales, act_rotations, act_opacities, leaves[4], leaves[5], empty, settings(cams_dev[vi]), False)
        if sparse:     # the union of the ranks' visible sets is formed on a side stream while the forward still blends
            visible, ready = rasterization.last_training_visibility(device, with_event=True)
            if overlap:
                xchg.begin(visible, ready, mode=scene.mode)
            elif compact:
                xchg.begin(visible, ready)
            else:
                exchange = parallel.begin_row_exchange(visible, ready=ready)
        loss = (image - target).abs().mean()
        loss.backward()      # with --exchange overlap the rasterizer's backward sums its gradients over the ranks range by range
        if overlap:
            exchanged_rows.append(xchg.rows_exchanged)
        elif compact:
            exchanged_rows.append(xchg.rows_published)
            gathered_bytes.append(xchg.bytes_gathered)
        elif sparse:
            exchanged_rows.append(parallel.finish_row_exchange([l.grad for l in leaves], exchange))
        elif dist is not None:
            parallel.allreduce_gradients([l.grad for l in leaves])
        return loss

    for s in range(warmup):
        step(s)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(device.index)
    sampler.start()
    time.sleep(0.25)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    e0.record()
    for s in range(warmup, warmup + steps):
        loss = step(s)
    e1.record()
    torch.cuda.synchronize()
    t1 = time.time()
    if dist is not None:
        dist.barrier()
    clocks = sampler.stop(t0, t1)
    ms = parallel.max_over_ranks(e0.elapsed_time(e1), device)
    exposed = None
    if compact:
        rasterization.set_backward_hook(None)
        counts = xchg.published_rows()
        if counts is not None:      # peer transport: bytes this rank read from the other ranks' buffers in the last step
            gathered_bytes = [sum(c for r, c in enumerate(counts) if r != rank) * parallel.kCompactRowBytes] * (warmup + 1)
        xchg.close()
    if overlap:
        rasterization.set_backward_hook(None)
        waits = xchg.exposed_ms(last=steps)
        exposed = parallel.max_over_ranks(float(np.mean(waits)) if waits else 0.0, device)
    if sparse:
        rasterization.track_training_visibility(False)
    n = scene.n
    row_bytes = (3 + 3 + 4 + 1 + 3 + 3 * scene.sh_rest.shape[1]) * 4
    grad_bytes = int(np.mean(gathered_bytes[warmup:])) if compact else int(np.mean(exchanged_rows[warmup:])) * row_bytes if sparse else n * row_bytes
    line = {"metric": "train-steps/s", "value": steps / (ms / 1000.0), "unit": "steps/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name.replace("config1", "config2 (fwd+bwd, L1, one view per GPU)"), "views_per_step": world,
                       "allreduce_bytes_per_rank": grad_bytes if world > 1 else 0,
                       "gradient_exchange": ("none" if (world == 1 and not sparse) else
                                             f"rows of the union of the ranks' visible Gaussians, summed range by range ({args.exchange_chunks} ranges{', per-tile pass split too' if args.exchange_split_pass else ''}) while the backward pass runs" if overlap else
                                             ("compact rows (64 B per Gaussian a rank's view kept), read from the peers' buffers over NVLink by the kernel that expands them" if compact_transport == "peer"
                                              else "compact rows (64 B per Gaussian a rank's view kept), all-gathered and expanded on every rank") if compact else
                                             "rows of the union of the ranks' visible Gaussians" if sparse else "dense tensors"),
                       "exchange_exposed_ms": exposed,
                       "views_per_s": world * steps / (ms / 1000.0), "views_of_a_step": "spread evenly over the orbit", "parallelism": f"view-partitioned x{world} + gradient all-reduce"},
            "clocks": clocks, "final_loss": float(loss.item())}
    if is_reference:
        line["impl"] = "reference"
    for l in leaves:
        l.grad = None
    return line


def train_leg_summary(line):
    """The training line folded into the `train` object of the default workload's JSON line."""
    cfg = line["config"]
    return {"metric": "train-steps/s", "steps_per_s": line["value"], "ms_per_step": line["ms_per_step"], "views_per_s": cfg["views_per_s"],
            "exchange": {"none": "none", "dense tensors": "dense"}.get(cfg["gradient_exchange"], "rows, overlapped with the backward" if "range by range" in cfg["gradient_exchange"]
                                                                       else "compact" if cfg["gradient_exchange"].startswith("compact") else "rows"),
            "exchange_exposed_ms": cfg.get("exchange_exposed_ms"),
            "allreduce_bytes_per_rank": cfg["allreduce_bytes_per_rank"], "n_gpus": line["n_gpus"], "steps": line["steps"], "warmup": line["warmup"],
            "workload": cfg["workload"], "clocks": line["clocks"], "final_loss": line["final_loss"]}


def main():
    args = parse_args()
    rank, world, local_rank = parallel.rank_world()
    if world != args.gpus and world > 1:
        args.gpus = world
    scene, workload_name = make_workload(args)

    import torch
    have_gpu = torch.cuda.is_available()
    ref_mod = None
    if args.impl == "reference":
        if args.reference_kind in ("auto", "cuda") and have_gpu:
            sys.path.insert(0, os.path.join(REPO, "tests"))
            import harness
            ref_mod = harness.reference()
        if ref_mod is None:
            if args.reference_kind == "cuda":
                if rank == 0:
                    print(json.dumps({"impl": "reference", "unavailable": "reference CUDA extension not built under baseline/_ref or no GPU"}), flush=True)
                return
            run_reference_cpu(args, scene, workload_name, rank, world)
            return
    if not have_gpu:
        raise SystemExit("bench.py: no CUDA device; the CUDA path has no CPU fallback")

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        # NCCL announces its version on standard output when its communicator is created (NCCL_DEBUG=VERSION and above):
        # create it here, with descriptor 1 pointed at standard error, so that the JSON line is the only line on stdout.
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist = parallel.init_process_group("nccl")
            dist.all_reduce(torch.zeros(1, device=device))
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)

    if ref_mod is not None:
        mod = ref_mod
    else:
        import htgs_b200.torch_bindings as mod
        from htgs_b200.torch_bindings import _C as our_C
        from htgs_b200 import _native

    tensors = [torch.from_numpy(np.ascontiguousarray(a)).to(device) for a in scene.arrays()]
    n_views = len(scene.views)
    cams_dev = [(torch.from_numpy(v.M).to(device), torch.from_numpy(v.VPM).to(device), torch.from_numpy(v.cam_position).to(device)) for v in scene.views]
    # per view ONE pinned host buffer (M, VPM, camera position = 35 floats): one host-to-device copy per frame
    cams_host = [torch.from_numpy(np.concatenate([v.M.reshape(-1), v.VPM.reshape(-1), v.cam_position.reshape(-1)]).astype(np.float32)).pin_memory()
                 for v in scene.views]
    v0 = scene.views[0]
    mode_enum = mod.RasterizerMode(scene.mode)

    def settings(cam):
        return mod.RasterizerSettings(M=cam[0], VPM=cam[1], cam_position=cam[2], mode=mode_enum, K=scene.K, active_sh_bases=scene.active_sh_bases,
                                      width=v0.width, height=v0.height, near_plane=v0.near_plane, far_plane=v0.far_plane, scale_modifier=1.0)

    if args.workload == "train":
        line = run_training(args, mod, ref_mod is not None, scene, tensors, cams_dev, settings, device, dist, rank, world, workload_name)
        if rank == 0:
            print(json.dumps(line), flush=True)
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return

    def train_leg():
        """Configuration 2 behind the render timing of the default workload: the other half of the metric (train-steps/s)."""
        if args.workload != "render" or args.no_train_leg:
            return None
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        tl = run_training(args, mod, ref_mod is not None, scene, tensors, cams_dev, settings, device, dist, rank, world, workload_name,
                          steps=args.train_steps or args.steps, warmup=max(args.warmup, 3))
        return train_leg_summary(tl)

    fast = args.workload == "render_fast"   # the relaxed-precision RGB-only entry point (`fast_rasterize`) of either implementation
    if fast:
        workload_name = workload_name.replace("config1", "config1 via fast_rasterize (relaxed precision, RGB only)")
    # Frames in flight.  This library's contexts are re-entrant (no global device state), so two frames can be in flight on
    # one GPU: the small kernels and the tail of one frame overlap the next frame's work.  Driver "async" (default): ONE host
    # thread queues frames on two CUDA streams through the non-blocking path (`set_deferred_checks`: htgs_render_async, status
    # checked one frame later).  Driver "threads": `--streams` host threads with blocking calls, one CUDA stream each.  The
    # reference keeps per-call state in module-global constant memory and a function-static stream
    # (rasterization/include/kernel_utils.cuh:10-12) and blocks in mid-frame, so its arm runs one frame at a time.
    driver = "async" if args.driver == "auto" else args.driver
    if driver == "threads":
        if args.streams > 0:
            n_lanes = args.streams
        else:
            try:
                host_threads = len(os.sched_getaffinity(0))
            except AttributeError:
                host_threads = os.cpu_count() or 1
            n_lanes = 2 if host_threads >= 3 * world else 1   # a lane's thread busy-waits on its stream: do not oversubscribe the host
    else:
        n_lanes = args.streams if args.streams > 0 else 2
    if ref_mod is not None:
        n_lanes = 1
    if n_lanes == 1:
        driver = "single"

    def render_any(cam):
        if fast:
            return mod.fast_rasterize(*tensors, settings(cam), True), None
        return mod.rasterize(*tensors, settings(cam), True, False)

    n_pix = v0.width * v0.height

    class Lane:
        """One host thread's share of the job: its CUDA stream, its copy-back stream and two alternating pinned buffers."""

        def __init__(self, own_stream: bool):
            self.stream = torch.cuda.Stream(device=device) if own_stream else torch.cuda.current_stream(device)
            self.copy_stream = torch.cuda.Stream(device=device)
            self.host_out = [(torch.empty((3, v0.height, v0.width), dtype=torch.float32).pin_memory(),
                              torch.empty((1, v0.height, v0.width), dtype=torch.float32).pin_memory(), torch.cuda.Event()) for _ in range(2)]
            self.count = 0
            self.launches = 0

        def resident(self, view_idx):
            render_any(cams_dev[view_idx])
            if ref_mod is None and not mod.rasterization.deferred_checks():
                self.launches += our_C.last_frame_info.kernel_launches

        def e2e(self, view_idx):
            # camera H2D from pinned memory -> rasterize -> image (+ depth) D2H into pinned memory; the copies back run on the
            # lane's second stream into two alternating pinned buffers, so that they overlap the next frame's kernels
            packed = cams_host[view_idx].to(device, non_blocking=True)
            cam = (packed[:16].view(4, 4), packed[16:32].view(4, 4), packed[32:35])
            image, depth = render_any(cam)
            h_img, h_depth, done = self.host_out[self.count % 2]
            self.count += 1
            done.synchronize()                       # the copy that used this pinned buffer two frames ago has finished
            self.copy_stream.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(self.copy_stream):
                h_img.copy_(image, non_blocking=True)
                if depth is not None:
                    h_depth.copy_(depth, non_blocking=True)
                done.record(self.copy_stream)
            image.record_stream(self.copy_stream)
            if depth is not None:
                depth.record_stream(self.copy_stream)

    # the reference launches on the legacy default stream whatever torch's current stream is: its arm is timed on that stream
    lanes = [Lane(own_stream=ref_mod is None) for _ in range(n_lanes)]
    launches = [0]

    def timed(kind, steps, warmup, sample_clocks=False, driver=driver, frame_marks=None):
        import threading
        n_lanes_used = 1 if driver == "single" else n_lanes
        timed_views = [vi for s in range(warmup, warmup + steps) for vi in parallel.step_view_indices(s, args.views_per_step, rank, world, n_views)]
        warm_views = [vi for s in range(warmup) for vi in parallel.step_view_indices(s, args.views_per_step, rank, world, n_views)]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        gate = threading.Barrier(n_lanes_used + 1)
        errors = []
        for lane in lanes:
            lane.launches = 0

        def lane_body(k):
            lane = lanes[k]
            fn = lane.resident if kind == "resident" else lane.e2e
            try:
                torch.cuda.set_device(device)
                with torch.cuda.stream(lane.stream):
                    # untimed: the views of the timed region once (either implementation grows its buffers / allocator pools), then the warm-up steps
                    for vi in timed_views[k::n_lanes_used] + warm_views[k::n_lanes_used]:
                        fn(vi)
                    lane.stream.synchronize()
                    lane.copy_stream.synchronize()
                    gate.wait()          # everybody is warm
                    gate.wait()          # the main thread has recorded the start event
                    lane.stream.wait_event(e0)
                    lane.launches = 0
                    for vi in timed_views[k::n_lanes_used]:
                        fn(vi)
                    lane.stream.wait_stream(lane.copy_stream)   # outstanding copies back belong to the timed region
            except Exception as exc:  # noqa: BLE001 - reported by the main thread
                errors.append(exc)
                gate.abort()

        def prepare():
            torch.cuda.synchronize()
            if dist is not None:
                dist.barrier()
            torch.cuda.synchronize()
            sampler = ClockSampler(local_rank) if sample_clocks else None
            if sampler:
                sampler.start()
                time.sleep(0.25)
            return sampler

        main_stream = torch.cuda.current_stream(device)
        if driver == "single":
            lane = lanes[0]
            fn = lane.resident if kind == "resident" else lane.e2e
            with torch.cuda.stream(lane.stream):
                for vi in timed_views + warm_views:
                    fn(vi)
            sampler = prepare()
            lane.launches = 0
            t0 = time.time()
            e0.record(main_stream)
            lane.stream.wait_event(e0)
            marks = []
            with torch.cuda.stream(lane.stream):
                for vi in timed_views:
                    fn(vi)
                    if frame_marks is not None:
                        marks.append(torch.cuda.Event(enable_timing=True))
                        marks[-1].record()
            main_stream.wait_stream(lane.stream)
            main_stream.wait_stream(lane.copy_stream)   # outstanding copies back belong to the timed region
            e1.record(main_stream)
            if frame_marks is not None:
                torch.cuda.synchronize()
                frame_marks.extend(a.elapsed_time(b) for a, b in zip([e0] + marks[:-1], marks))
        elif driver == "async":
            # one host thread, frames alternate between the lanes' streams; no call waits for the GPU, a frame's status is
            # checked when its stream is used again (two frames later) and, for the last ones, by frame_results()
            def sweep(views, count_launches):
                for i, vi in enumerate(views):
                    lane = lanes[i % n_lanes_used]
                    with torch.cuda.stream(lane.stream):
                        (lane.resident if kind == "resident" else lane.e2e)(vi)
                infos = mod.rasterization.frame_results(device)
                if count_launches:
                    # every frame of the sweep launches the same kernels: count one frame's and scale
                    per_frame = max((fi.kernel_launches for fi in infos), default=0)
                    lanes[0].launches = per_frame * len(views)
                return infos

            for lane in lanes[:n_lanes_used]:      # first pass with blocking calls: buffers grow to what these views need
                with torch.cuda.stream(lane.stream):
                    for vi in timed_views + warm_views:
                        (lane.resident if kind == "resident" else lane.e2e)(vi)
            mod.rasterization.set_deferred_checks(True)
            try:
                sweep(warm_views + timed_views[: 2 * n_lanes_used], False)
                sampler = prepare()
                t0 = time.time()
                e0.record(main_stream)
                for lane in lanes[:n_lanes_used]:
                    lane.stream.wait_event(e0)
                infos = sweep(timed_views, True)
                for lane in lanes[:n_lanes_used]:
                    main_stream.wait_stream(lane.stream)
                    main_stream.wait_stream(lane.copy_stream)
                e1.record(main_stream)
                if any(fi.reruns for fi in infos):
                    raise RuntimeError("a frame of the timed region was re-rendered by its deferred check")
            finally:
                mod.rasterization.set_deferred_checks(False)
        else:
            threads = [threading.Thread(target=lane_body, args=(k,)) for k in range(n_lanes_used)]
            for th in threads:
                th.start()
            try:
                gate.wait()
                sampler = prepare()
                t0 = time.time()
                e0.record(main_stream)
                gate.wait()
            except threading.BrokenBarrierError:
                sampler = None
                t0 = time.time()
            for th in threads:
                th.join()
            if errors:
                raise errors[0]
            for lane in lanes:
                main_stream.wait_stream(lane.stream)
            e1.record(main_stream)
        torch.cuda.synchronize()
        t1 = time.time()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        clocks = sampler.stop(t0, t1) if sampler else None
        launches[0] = sum(lane.launches for lane in lanes)
        ms = parallel.max_over_ranks(e0.elapsed_time(e1), device)
        return ms, clocks

    ref_frames = [] if ref_mod is not None else None   # per-frame times of the reference arm (it runs one frame at a time anyway)
    ms_total, clocks = timed("resident", args.steps, args.warmup, sample_clocks=True, frame_marks=ref_frames)
    frames_total = args.steps * args.views_per_step * world
    value = frames_total / (ms_total / 1000.0)
    timed_launches = launches[0] * world
    ms_e2e, _ = timed("e2e", args.steps, args.warmup)
    e2e_value = frames_total / (ms_e2e / 1000.0)

    line = {
        "metric": "frames/s", "value": value, "unit": "frames/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": workload_name, "views_per_step_per_gpu": args.views_per_step, "parallelism": f"view-partitioned x{world}",
                   "l2": "per-frame working set (708 MB scene + >300 MB per-Gaussian records) exceeds the 126 MB L2; no explicit flush",
                   "scene_residency": "scene resident in HBM; per-frame inputs are the camera matrices",
                   "frames_in_flight": n_lanes, "frame_driver": {"async": "one host thread, two CUDA streams, non-blocking calls (deferred status checks)",
                                                                    "threads": f"{n_lanes} host threads with blocking calls", "single": "one host thread, blocking calls"}[driver]},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "frames/s", "h2d_bytes_per_step": args.views_per_step * (16 + 16 + 3) * 4,
                "d2h_bytes_per_step": args.views_per_step * n_pix * 4 * (3 if fast else 4), "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": timed_launches,
    }

    if ref_mod is None and n_lanes > 1:
        # the same job with one frame in flight (one host thread, one stream, blocking calls), and with the other two-frame driver
        per_frame = []
        ms_1, _ = timed("resident", args.steps, args.warmup, driver="single", frame_marks=per_frame)
        ms_1e, _ = timed("e2e", args.steps, args.warmup, driver="single")
        line["one_frame_in_flight"] = {"value": frames_total / (ms_1 / 1000.0), "e2e": frames_total / (ms_1e / 1000.0), "unit": "frames/s",
                                       "frame_ms": {"p10": float(np.percentile(per_frame, 10)), "p50": float(np.percentile(per_frame, 50)),
                                                    "p90": float(np.percentile(per_frame, 90)), "frames": len(per_frame)}}
        other = "threads" if driver == "async" else "async"
        try:
            host_threads = len(os.sched_getaffinity(0))
        except AttributeError:
            host_threads = os.cpu_count() or 1
        if other == "async" or host_threads >= 3 * world:
            ms_o, _ = timed("resident", args.steps, args.warmup, driver=other)
            ms_oe, _ = timed("e2e", args.steps, args.warmup, driver=other)
            line["other_driver"] = {"driver": other, "value": frames_total / (ms_o / 1000.0), "e2e": frames_total / (ms_oe / 1000.0), "unit": "frames/s"}

    if ref_mod is not None:
        line["frame_ms"] = {"p10": float(np.percentile(ref_frames, 10)), "p50": float(np.percentile(ref_frames, 50)),
                            "p90": float(np.percentile(ref_frames, 90)), "frames": len(ref_frames)}
        line.update({"impl": "reference", "reference_kind": "cuda-extension (unmodified HTGSCudaBackend built for sm_100a under baseline/_ref)",
                     "gpu_launches": 0,
                     "cpu_baseline": {"value": None, "unit": "frames/s", "cores": 0, "kind": "reference",
                                      "sample": "not a CPU run: this arm executed the reference's CUDA extension (it has no CPU path)"}})
        line["train"] = train_leg()
        if rank == 0:
            print(json.dumps(line), flush=True)
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- per-stage device times, statistics and rooflines (outside the timed regions) ---------------
    ctx = _native.context(local_rank)
    lib = _native.lib()
    import ctypes
    probe_views = [parallel.step_view_indices(args.warmup + (i * args.steps) // 8, args.views_per_step, rank, world, n_views)[i % args.views_per_step] for i in range(8)]
    lib.htgs_set_profiling(ctx, 1)
    stage = np.zeros((len(probe_views), 7), np.float64)
    buf = (ctypes.c_float * 7)()
    infos = []
    for _ in range(2):   # second round is the one kept (warm)
        for i, vi in enumerate(probe_views):
            render_any(cams_dev[vi])
            lib.htgs_get_stage_ms(ctx, buf)
            stage[i] = np.array(buf[:], np.float64)
    lib.htgs_set_profiling(ctx, 0)
    lib.htgs_set_collect_stats(ctx, 1)
    for vi in probe_views:
        mod.rasterize(*tensors, settings(cams_dev[vi]), True, False)   # the exact kernel counts candidates / accepted fragments
        fi = our_C.last_frame_info
        infos.append((fi.n_instances, fi.n_visible, fi.candidate_pairs, fi.accepted_fragments, fi.key_bytes, fi.end_bit, fi.warp_trips, fi.warp_trips_inserting,
                      fi.lane_insertions))
    lib.htgs_set_collect_stats(ctx, 0)
    infos = np.array(infos, np.float64)
    I, n_vis, cand, acc = infos[:, 0].mean(), infos[:, 1].mean(), infos[:, 2].mean(), infos[:, 3].mean()
    key_bytes, end_bit = int(infos[0, 4]), int(infos[0, 5])
    stage_ms = stage.mean(axis=0)
    names = ["preprocess", "scan", "emit", "sort", "ranges", "blend", "total"]
    hbm_peak, peak_kind = load_measured_peaks()
    n = scene.n
    sh_active = scene.active_sh_bases
    n_tiles = ((v0.width + 7) // 8) * ((v0.height + 7) // 8)
    pre_bytes = n * 44 + n_vis * (12 + 12 * (sh_active - 1)) + n_vis * 84 + n * 4
    passes_ref = (end_bit + 7) // 8
    bin_bytes = I * (key_bytes + 4) + passes_ref * 2 * I * (key_bytes + 4) + I * key_bytes + 8 * n_tiles
    pairs = 64.0 * I
    blend_flops = pairs * 54 + acc * (60 + 7 * scene.K)
    sm_mhz = (clocks or {}).get("sm_mhz") or 1965.0
    sm_count = torch.cuda.get_device_properties(device).multi_processor_count
    fp32_peak_tflops = sm_count * 128 * 2 * sm_mhz * 1e6 / 1e12
    blend_ms = stage_ms[5]
    bin_ms = stage_ms[1] + stage_ms[2] + stage_ms[3] + stage_ms[4]
    line["roofline"] = {
        "kernel": f"blend_fast_kernel<{MODE_NAMES[scene.mode]},{scene.K}>" if fast else f"blend_kernel<{MODE_NAMES[scene.mode]},{scene.K}>", "bound": "fp32",
        "achieved": blend_flops / (blend_ms * 1e-3) / 1e12, "peak": fp32_peak_tflops, "unit": "TFLOP/s",
        "frac": blend_flops / (blend_ms * 1e-3) / 1e12 / fp32_peak_tflops,
        "peak_source": f"{sm_count} SMs x 128 FP32 lanes x 2 x {sm_mhz:.0f} MHz (SM clock sampled during the timed region); no tensor-core work on this path",
        "traffic": 24.0 * I, "traffic_note": "DRAM bytes per launch = 24 B x instances, scaled from an ncu capture at 1 M Gaussians (44 MB read + 1.5 MB written for 1.89 M instances; the evaluation records are read once, re-use hits L2)",
        "ms": blend_ms,
        # the same kernel seen as a memory stream (what it must read and write: 84 B per instance record + 16 B per pixel):
        # it sits far below the HBM roofline, which is why the FP32 issue rate above is the bound that is reported
        "hbm_view": {"bound": "hbm", "bytes": I * 84.0 + n_pix * 16.0, "achieved": (I * 84.0 + n_pix * 16.0) / (blend_ms * 1e-3) / 1e9,
                     "peak": hbm_peak, "unit": "GB/s", "frac": (I * 84.0 + n_pix * 16.0) / (blend_ms * 1e-3) / 1e9 / hbm_peak,
                     "peak_source": f"{peak_kind} copy bandwidth"},
        "insertion_chain": None if (fast or scene.mode != 0 or not infos[:, 6].mean()) else {
            "warp_trips": float(infos[:, 6].mean()), "share_of_trips_with_an_insertion": float(infos[:, 7].mean() / infos[:, 6].mean()),
            "inserting_lanes_per_such_trip": float(infos[:, 8].mean() / max(infos[:, 7].mean(), 1.0)),
            "note": "the K-level chain sits behind a per-lane branch, so a warp runs it only when one of its lanes inserts"},
        "algorithmic": {"pairs": pairs, "accepted_fragments": acc, "candidate_pairs": cand, "flops": blend_flops,
                        "formula": "pairs*54 + accepted*(60+7K), the reference algorithm's work (every pixel of a tile tests every instance of the tile)"},
    }
    line["roofline_hbm"] = [
        {"kernel": "preprocess_kernel", "bound": "hbm", "achieved": pre_bytes / (stage_ms[0] * 1e-3) / 1e9, "peak": hbm_peak, "unit": "GB/s",
         "frac": pre_bytes / (stage_ms[0] * 1e-3) / 1e9 / hbm_peak, "peak_source": f"{peak_kind} copy bandwidth", "ms": stage_ms[0], "bytes": pre_bytes},
        {"kernel": "binning (scan+emit+radix sort+ranges)", "bound": "hbm", "achieved": bin_bytes / (bin_ms * 1e-3) / 1e9, "peak": hbm_peak, "unit": "GB/s",
         "frac": bin_bytes / (bin_ms * 1e-3) / 1e9 / hbm_peak, "peak_source": f"{peak_kind} copy bandwidth", "ms": bin_ms, "bytes": bin_bytes,
         "note": "bytes of the reference algorithm (8-bit digits); this implementation needs fewer passes"},
    ]
    line["stages_ms"] = {k: float(v) for k, v in zip(names, stage_ms)}
    line["frame_stats"] = {"n_instances": I, "n_visible": n_vis, "key_bytes": key_bytes, "end_bit": end_bit}

    line["train"] = train_leg()
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        fps, cores, sample = cpu_port_fps(scene, args.cpu_sample_views)
        line["cpu_baseline"] = {"value": fps, "unit": "frames/s", "cores": cores, "kind": "port", "sample": sample}
    else:
        line["cpu_baseline"] = None
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
