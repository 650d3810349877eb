"""Throughput of the Visual Mesh hot path on B200s, with the reference CPU engine timed beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config 1] [--impl ours|reference]

A step is one pass of the hot path (device-side lookup, projection, compaction, neighbour remap, image sampling, all
graph-convolution layers) over one batch of synthetic frames; the headline workload is configuration 1: 64 seeded
1280x1024 RGBA frames, Ring6/Sphere mesh at h = 1.2 m, equidistant lens with distortion, 8-layer network. Rank 0
prints one JSON line:

  value         frames/s over all GPUs with the frames already resident in HBM and results left in HBM
  e2e           frames/s through the C ABI with frames in pinned HOST memory and results copied back to the host;
                copy_bound_ms is the time the same bytes take as bare copies (all ranks at once, no kernels)
  roofline      the dominant kernel against the measured HBM bandwidth
  cpu_baseline  the reference CPU engine on this box's host cores, on a bounded sample of the same frames
  sustained     the device-resident step run back to back for a few seconds, with the clocks seen
  configs       (one GPU) the other benchmark configurations, and (any N) configuration 4's height-mixed stream dealt
                frame i -> GPU i mod N
  parity        (one GPU) frames within tolerance of the reference CPU engine / frames, per configuration
  config.result_digest   sha256 of rank 0's results for frames 0..63 of the seeded stream: the same at every N

With N > 1 (launched by torchrun, one rank per GPU) every rank runs the same per-GPU batch on its own frames; frames
are independent, so there is no collective on the data path - only a barrier and a max over ranks around the timing.
`--impl reference` times the reference's own CPU engine (oracle/_ref, the unmodified reference compiled in place) with
one engine instance per host core, the pattern of example/benchmark.cpp:86-101,142.
"""
import argparse
import hashlib
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

import numpy as np  # noqa: E402

from visualmesh_b200 import sharding  # noqa: E402
from visualmesh_b200 import workloads as W  # noqa: E402

# VMCUDA_BLOCKING_SYNC exported by the caller applies to every engine; otherwise the bench decides per engine (Arm)
USER_SET_BLOCKING_SYNC = "VMCUDA_BLOCKING_SYNC" in os.environ

# DRAM traffic per row of the dominant kernels from their ncu captures (dram__bytes_read + dram__bytes_write over the
# rows of the captured launch); traffic grows in proportion to the rows, so it is scaled to the bench's launches.
NCU_TRAFFIC_BYTES_PER_ROW = {
    (16, 16): 110.6,  # profiles/graph_conv_staged_16x16_cfg1_16frames.md: 122.6 MB over 1,108,261 rows
    (32, 32): 250.4,  # profiles/graph_conv_tc_tmem_32x32_cfg3_1frame.md: 233.3 MB over 931,718 rows
}


def _kernel_of_layer(cin, cout):
    """Which kernel the engine's default policy runs a gather layer on (visualmesh_b200/csrc/engine.cu, run_network)."""
    if cin == 16 and cout in (8, 16, 32):
        return "st::k_graph_conv_mma (shared-memory windows, ldmatrix gather, mma.sync)"
    if cin in (16, 32) and cout in (16, 32) and cin * cout >= 512:
        return "tc::k_graph_conv_tc_tmem (tcgen05, A operand in tensor memory)"
    return "k_graph_conv_cw (FFMA)"


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.samples = []
        self.proc = None
        self.device_index = device_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.device_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append((time.time(), parts))

    def stop(self):
        if self.proc is None:
            return
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()

    def summary(self, windows):
        """windows: [(t0, t1)] host-clock intervals. Samples inside them are "under load"; a region shorter than the
        sampling period takes the samples closest to it."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        inside = [p for t, p in self.samples if any(a <= t <= b + 0.12 for a, b in windows)]
        if not inside and self.samples and windows:
            mid = 0.5 * (windows[0][0] + windows[-1][1])
            inside = [p for _, p in sorted(self.samples, key=lambda tp: abs(tp[0] - mid))[:2]]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in inside:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except ValueError:
                continue
            for name, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def _physical_device(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        ids = [v for v in vis.split(",") if v != ""]
        if local_rank < len(ids) and ids[local_rank].isdigit():
            return int(ids[local_rank])
    return local_rank


# ---------------------------------------------------------------------------------------------------------------------
# reference arm / CPU baseline
# ---------------------------------------------------------------------------------------------------------------------

_REF_MESHES, _REF_IMAGES = {}, {}


def _cpu_reference_run(wl, frames, n_threads):
    """One pass of the reference CPU engine over `frames` with n_threads workers; mesh construction and image
    generation are outside the timed call. Returns (seconds, points, kind, threads)."""
    import refharness as R
    if R.available():
        ms = [_REF_MESHES.setdefault(fr.mesh.key(), R.RefMesh(fr.mesh)) for fr in frames]
        images = [_REF_IMAGES.setdefault(fr.image_seed, fr.image()) for fr in frames]
        secs, points = R.run_stream(ms, [fr.Hoc for fr in frames], [fr.lens for fr in frames], images,
                                    [fr.format for fr in frames], wl.network, n_threads)
        return secs, points, "reference", n_threads
    # no compiled reference on this machine: the single-threaded plain-C restatement
    import oracle as O
    from visualmesh_b200.engine import Mesh
    meshes = {}
    t0 = time.perf_counter()
    points = 0
    for fr in frames:
        m = meshes.setdefault(fr.mesh.key(), Mesh.from_spec(fr.mesh))
        ranges = O.lookup(m.rays, (m.bsp_ranges, m.bsp_children, m.bsp_cones), fr.Hoc, fr.lens)
        out = O.classify(m.rays, m.neighbours, ranges, wl.network, fr.Hoc, fr.lens, fr.image(), fr.format)
        points += len(out["global_indices"])
    return time.perf_counter() - t0, points, "port", 1


def run_reference(args, rank, world):
    if rank != 0:
        return
    wl = W.config(args.config, seed=args.seed, n_frames=max(args.frames, 1))
    cores = os.cpu_count() or 1
    frames = wl.frames[:args.frames]  # the same frames per step as rank 0 of the other arm
    for _ in range(args.warmup and 1):
        _cpu_reference_run(wl, frames[:min(len(frames), cores)], cores)
    total_s, total_pts, kind, used = 0.0, 0, "reference", cores
    for _ in range(args.steps):
        s, pts, kind, used = _cpu_reference_run(wl, frames, cores)
        total_s += s
        total_pts += pts
    fps = args.steps * len(frames) / total_s
    line = {
        "impl": "reference", "metric": "frames/s", "value": fps, "unit": "frames/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total_s / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "nodes_per_s": total_pts / total_s,
        "config": _config_block(wl, len(frames), total_pts / args.steps / len(frames), 1,
                                note="reference CPU engine, one fresh engine instance per frame, one worker per host core"),
        "cpu_baseline": {"value": fps, "unit": "frames/s", "cores": used, "kind": kind,
                         "sample": f"{len(frames)} frames of {wl.name} per step"},
        "e2e": {"value": fps, "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def _config_block(wl, per_gpu, nodes_per_frame, world, note=None):
    block = {"workload": wl.name + ": " + wl.description, "frames_per_gpu_per_step": per_gpu,
             "on_screen_nodes_per_frame": nodes_per_frame, "lookup": "device BSP walk", "l2": "inputs_larger_than_l2",
             "distortion": "k_px = (k1/W^2, k2/W^4)", "parallelism": f"frame-sharded x{world}"}
    if note:
        block["note"] = note
    return block


# ---------------------------------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------------------------------

class Arm:
    """One workload on one GPU: its frames once in pinned host memory (the end-to-end mode) and once in HBM (the
    device-resident mode), an engine, and the two timed loops."""

    def __init__(self, wl, frames, device, instances, sleepy_e2e=False):
        import torch
        from visualmesh_b200.engine import Engine, FrameInput, Mesh
        self.torch, self.wl, self.frames, self.device = torch, wl, frames, device

        def make_engine(sleepy):
            # an engine reads VMCUDA_BLOCKING_SYNC when it is created; a value the user exported is left alone
            if USER_SET_BLOCKING_SYNC:
                return Engine(wl.network, device=device)
            os.environ["VMCUDA_BLOCKING_SYNC"] = "1" if sleepy else "0"
            try:
                return Engine(wl.network, device=device)
            finally:
                os.environ.pop("VMCUDA_BLOCKING_SYNC", None)

        # the device-resident loop has one host thread per GPU: its waits always spin
        self.engine = make_engine(False)
        self.meshes = {}
        for fr in frames:
            if fr.mesh.key() not in self.meshes:
                self.meshes[fr.mesh.key()] = Mesh.from_spec(fr.mesh)
        self.sizes = [fr.image_bytes for fr in frames]
        starts = np.concatenate([[0], np.cumsum([(s + 255) // 256 * 256 for s in self.sizes])]).astype(np.int64)
        self.host = torch.empty(int(starts[-1]), dtype=torch.uint8, pin_memory=True)
        host_np = self.host.numpy()
        for i, fr in enumerate(frames):
            host_np[starts[i]:starts[i] + self.sizes[i]] = fr.image()
        self.dev = self.host.cuda(non_blocking=False)
        torch.cuda.synchronize()
        self.host_frames = [FrameInput(self.meshes[fr.mesh.key()], fr.Hoc, fr.lens,
                                       host_np[starts[i]:starts[i] + self.sizes[i]], fr.format, None)
                            for i, fr in enumerate(frames)]
        dev_frames = [FrameInput(self.meshes[fr.mesh.key()], fr.Hoc, fr.lens, self.dev.data_ptr() + int(starts[i]),
                                 fr.format, None, image_on_device=True) for i, fr in enumerate(frames)]
        self.dev_batch = self.engine.prepare_batch(dev_frames)
        # end-to-end mode: `instances` engine instances, one host thread each, split the batch between them and run
        # their steps back to back - the reference's own advice for its GPU engines (readme/inference.md:70-77,
        # example/benchmark.cpp:86-101, :133): while one instance waits for its last copies another uploads
        n_inst = max(1, min(instances, len(frames)))
        # (with many ranks on a box with few cores these threads' waits sleep instead of spinning: engines of their own)
        self.engines = ([make_engine(True) for _ in range(n_inst)] if sleepy_e2e
                        else [self.engine] + [make_engine(False) for _ in range(n_inst - 1)])
        parts = [sharding.shard(self.host_frames, i, n_inst) for i in range(n_inst)]
        self.batches = [eng.prepare_batch(part) for eng, part in zip(self.engines, parts)]
        self.d2h_bytes = 0

    def stage_names(self):
        """The engine's stage name of every dense layer, in order (graph_conv_<cin>x<cout> for the first layer of a
        group, dense_<cin>x<cout> for the ones that follow it)."""
        names, width = [], 4
        for group in self.wl.network:
            for i, layer in enumerate(group):
                cout = layer.biases.shape[0]
                names.append(("graph_conv_" if i == 0 else "dense_") + f"{width}x{cout}")
                width = cout
        return names

    def warm(self, n):
        for _ in range(n):
            self.engine.run_prepared(self.dev_batch, results_on_device=True, time_stages=True, raw=True)
            self.engine.run_prepared(self.dev_batch, results_on_device=True, raw=True)
        for eng, b in zip(self.engines, self.batches):
            for _ in range(n):
                eng.run_prepared(b, raw=True)

    def run_device(self, steps):
        """The timed region of `value`: (device ms, points, kernel launches, (wall t0, t1))."""
        engine = self.engine
        launches0, points = engine.launch_count(), 0
        w0 = time.time()
        engine.timer_start()
        for _ in range(steps):
            res = engine.run_prepared(self.dev_batch, results_on_device=True, raw=True)
            points += int(res.offsets[res.n_frames])
        device_ms = engine.timer_stop()
        return device_ms, points, engine.launch_count() - launches0, (w0, time.time())

    def run_device_stages(self, steps):
        """The same steps once more with an event pair around every kernel (which serialises the engine's streams, so
        this region is not the one `value` comes from): (stage ms totals, stage launch counts, (wall t0, t1))."""
        engine = self.engine
        stage_total, stage_launches = {}, {}
        w0 = time.time()
        for _ in range(steps):
            engine.run_prepared(self.dev_batch, results_on_device=True, time_stages=True, raw=True)
            for name, ms in engine.stage_times():
                stage_total[name] = stage_total.get(name, 0.0) + ms
                stage_launches[name] = stage_launches.get(name, 0) + 1
        return stage_total, stage_launches, (w0, time.time())

    def run_device_for(self, seconds):
        """The device-resident step back to back for at least `seconds`: (device ms, steps, (wall t0, t1))."""
        engine, steps = self.engine, 0
        w0 = time.time()
        engine.timer_start()
        while time.time() - w0 < seconds:
            for _ in range(20):
                engine.run_prepared(self.dev_batch, results_on_device=True, raw=True)
            steps += 20
        device_ms = engine.timer_stop()
        return device_ms, steps, (w0, time.time())

    def run_e2e(self, steps):
        """(seconds, kernel launches, (wall t0, t1)); sets d2h_bytes (per step)."""
        d2h_parts = [0] * len(self.engines)

        def worker(i):
            for _ in range(steps):
                res = self.engines[i].run_prepared(self.batches[i], raw=True)
                n_pts = int(res.offsets[res.n_frames])
                n_rows = n_pts + res.n_frames
                d2h_parts[i] = (n_pts * (8 + 4) + n_rows * 4 * res.n_neighbours + n_rows * 4 * res.n_classes
                                + 4 * res.n_frames)

        launches0 = sum(eng.launch_count() for eng in self.engines)
        t1, w0 = time.perf_counter(), time.time()
        self.engine.timer_start()
        workers = [threading.Thread(target=worker, args=(i,)) for i in range(len(self.engines))]
        for w in workers:
            w.start()
        for w in workers:
            w.join()
        device_ms = self.engine.timer_stop()
        wall = time.perf_counter() - t1
        self.d2h_bytes = sum(d2h_parts)
        # results are complete on the host when the last worker returns: the host clock is the honest one here
        seconds = max(device_ms * 1e-3 if len(self.engines) == 1 else 0.0, wall)
        return seconds, sum(eng.launch_count() for eng in self.engines) - launches0, (w0, time.time())

    def copy_bound(self, steps, chunk_frames=16):
        """Seconds per step of the bare copies of one end-to-end step: every chunk's frames host -> device on one stream
        and a result-sized block device -> host on another, pinned memory, no kernels."""
        torch = self.torch
        n_chunks = max(1, (len(self.frames) + chunk_frames - 1) // chunk_frames)
        h2d = int(sum(self.sizes))
        d2h = max(int(self.d2h_bytes), 1)
        src = self.host[:h2d]
        dst = torch.empty(h2d, dtype=torch.uint8, device="cuda")
        back_dev = torch.empty(d2h, dtype=torch.uint8, device="cuda")
        back_host = torch.empty(d2h, dtype=torch.uint8, pin_memory=True)
        up, down = torch.cuda.Stream(), torch.cuda.Stream()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

        def step():
            for c in range(n_chunks):
                lo, hi = h2d * c // n_chunks, h2d * (c + 1) // n_chunks
                with torch.cuda.stream(up):
                    dst[lo:hi].copy_(src[lo:hi], non_blocking=True)
                lo, hi = d2h * c // n_chunks, d2h * (c + 1) // n_chunks
                with torch.cuda.stream(down):
                    back_host[lo:hi].copy_(back_dev[lo:hi], non_blocking=True)

        step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            step()
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / steps

    def digest(self, n_frames=64):
        """sha256 over the four result arrays (and the offsets) of the first n_frames frames, through the C ABI."""
        res = self.engine.run_batch(self.host_frames[:n_frames])
        h = hashlib.sha256()
        h.update(np.ascontiguousarray(res.offsets).tobytes())
        for f in range(res.n_frames):
            fr = res.frame(f, copy=False)
            for a in (fr.pixel_coordinates, fr.global_indices, fr.neighbourhood, fr.classifications):
                h.update(np.ascontiguousarray(a).tobytes())
        return h.hexdigest()

    def close(self):
        for eng in self.engines:
            eng.close()


def _roofline(arm, stage_total, stage_launches, rows_per_step, steps):
    """The graph-convolution layer that takes the most device time, as algorithmic bytes over its CUDA-event time."""
    conv = {k: v for k, v in stage_total.items() if k.startswith("graph_conv")}
    top = max(conv, key=conv.get)
    peak, peak_kind = _peaks()
    N = arm.wl.n_neighbours
    cin, cout = [int(v) for v in top.split("_")[-1].split("x")]
    layers_with_name = sum(1 for n in arm.stage_names() if n == top)
    bytes_per_row = 4 * cin + 4 * N + 4 * cout  # each array touched once; neighbour re-reads are expected L2 hits
    rows_total = rows_per_step * steps * layers_with_name
    top_s = 1e-3 * stage_total[top]
    achieved = bytes_per_row * rows_total / top_s / 1e9
    gpu_ms_total = sum(stage_total.values())
    return {"bound": "hbm", "kernel": f"graph_conv {cin}->{cout}: " + _kernel_of_layer(cin, cout),
            "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": f"of {peak_kind}",
            "traffic": (NCU_TRAFFIC_BYTES_PER_ROW[(cin, cout)] * rows_total / stage_launches[top])
            if (cin, cout) in NCU_TRAFFIC_BYTES_PER_ROW else None,
            "algorithmic_bytes_per_launch": bytes_per_row * rows_total / stage_launches[top],
            "avg_launch_ms": stage_total[top] / stage_launches[top],
            "fp32_tflops": 2.0 * (N + 1) * cin * cout * rows_total / top_s / 1e12,
            "share_of_gpu_time": stage_total[top] / gpu_ms_total}


def _other_config(cfg, args, local_rank, parity):
    """One of the other benchmark configurations on one GPU: device-resident and end-to-end frames/s, its dominant
    kernel, and the reference CPU engine's rate on the same box (from the parity run over the same configuration)."""
    n = 64  # frames per step, as for the headline (the configurations' own 1 / 32 / 32 frames repeat their generator)
    wl = W.config(cfg, seed=args.seed, n_frames=n)
    arm = Arm(wl, wl.frames, local_rank, args.instances)
    arm.warm(3)
    steps = 5 if cfg != 3 else 2
    device_ms, points, _, _ = arm.run_device(steps)
    stage_total, stage_launches, _ = arm.run_device_stages(steps)
    e2e_s, _, _ = arm.run_e2e(steps)
    rows_per_step = points / steps + n
    roof = _roofline(arm, stage_total, stage_launches, rows_per_step, steps)
    out = {"config": wl.name, "workload": wl.description, "frames_per_step": n,
           "value": n * steps / (device_ms * 1e-3), "unit": "frames/s", "nodes_per_s": points / (device_ms * 1e-3),
           "ms_per_step": device_ms / steps,
           "e2e": {"value": n * steps / e2e_s, "unit": "frames/s", "h2d_bytes_per_step": int(sum(arm.sizes)),
                   "d2h_bytes_per_step": int(arm.d2h_bytes)},
           "dominant_kernel": {"kernel": roof["kernel"], "frac": roof["frac"], "achieved_gbs": roof["achieved"],
                               "share_of_gpu_time": roof["share_of_gpu_time"]}}
    if parity and parity.get("reference_seconds"):
        out["cpu_baseline"] = {"value": parity["frames"] / parity["reference_seconds"], "unit": "frames/s",
                               "cores": min(os.cpu_count() or 1, parity["frames"]), "kind": "reference",
                               "sample": f"the {parity['frames']} frames of the parity check, one pass"}
    arm.close()
    return out


def run_ours(args, rank, world, local_rank):
    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU fallback")
    # several ranks' engine threads on a box with few cores: let the waits sleep instead of spinning
    cores = os.cpu_count() or 1
    sleepy_e2e = (os.environ.get("VMCUDA_BLOCKING_SYNC") == "1") if USER_SET_BLOCKING_SYNC else world * (args.instances + 1) > cores // 2
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        return sharding.max_over_ranks(dist, x, "cuda")

    def sum_over_ranks(x):
        return sharding.sum_over_ranks(dist, x, "cuda")

    sampler = ClockSampler(_physical_device(local_rank))
    sampler.start()
    per_gpu = args.frames
    wl = W.config(args.config, seed=args.seed, n_frames=per_gpu * world)
    frames = sharding.shard(wl.frames, rank, world)  # rank r takes its contiguous slice of the seeded stream
    arm = Arm(wl, frames, local_rank, args.instances, sleepy_e2e)

    # ---- device-resident arm: `value`, per-kernel times for the roofline ----
    warm = max(args.warmup, 3)
    arm.warm(warm)
    barrier()
    t0 = time.perf_counter()
    device_ms, points, launches, win_dev = arm.run_device(args.steps)
    wall = time.perf_counter() - t0
    barrier()
    stage_total, stage_launches, win_stages = arm.run_device_stages(args.steps)
    barrier()
    elapsed = max_over_ranks(device_ms * 1e-3)  # CUDA events on the engine's own stream, max over ranks
    total_frames = per_gpu * world * args.steps
    total_points = sum_over_ranks(points)
    value = total_frames / elapsed
    rows_per_step = points / args.steps + per_gpu  # one off-screen row per frame

    # ---- end-to-end arm: pinned host frames in, results back on the host, copies inside the timed region ----
    barrier()
    e2e_s, e2e_launches, win_e2e = arm.run_e2e(args.steps)
    e2e_elapsed = max_over_ranks(e2e_s)
    barrier()
    e2e_value = total_frames / e2e_elapsed
    launches += e2e_launches
    # the bare copies of the same bytes, every rank at once: what the box's host-device path gives without any kernel
    barrier()
    copy_s = max_over_ranks(arm.copy_bound(max(2, min(args.steps, 5)))) if not args.quick else None
    barrier()

    # ---- sustained: the same device-resident step back to back for seconds ----
    sustained = None
    if args.sustained_seconds > 0 and not args.quick:
        barrier()
        s_ms, s_steps, win_s = arm.run_device_for(args.sustained_seconds)
        s_elapsed = max_over_ranks(s_ms * 1e-3)
        barrier()
    sampler.stop()
    clocks = sampler.summary([win_dev, win_stages, win_e2e])
    if args.sustained_seconds > 0 and not args.quick:
        c = sampler.summary([win_s])
        s_value = per_gpu * world * s_steps / s_elapsed
        sustained = {"value": s_value, "unit": "frames/s", "seconds": s_elapsed, "steps": s_steps,
                     "sm_mhz_median": c["sm_mhz"], "sm_max_mhz": c["sm_max_mhz"], "reasons": c["reasons"],
                     "samples": c.get("samples")}
        if c["sm_mhz"] and c["sm_max_mhz"] and c["sm_mhz"] < 0.97 * c["sm_max_mhz"]:
            sustained["value_at_max_clock"] = s_value * c["sm_max_mhz"] / c["sm_mhz"]

    # ---- roofline of the dominant kernel ----
    roofline = _roofline(arm, stage_total, stage_launches, rows_per_step, args.steps)
    gpu_ms_total = sum(stage_total.values())
    stages = [{"kernel": k, "ms_per_step": v / args.steps, "launches_per_step": stage_launches[k] / args.steps,
               "share": v / gpu_ms_total} for k, v in sorted(stage_total.items(), key=lambda kv: -kv[1])]

    # ---- the same answers at every N: rank 0 always holds frames 0..63 of the seeded stream ----
    digest = arm.digest(min(64, len(frames))) if rank == 0 and not args.quick else None
    h2d_bytes, d2h_bytes = int(sum(arm.sizes)), int(arm.d2h_bytes)
    arm.close()
    del arm
    torch.cuda.empty_cache()

    # ---- configuration 4 as it is defined: ONE height-mixed stream dealt frame i -> GPU i mod N (strong scaling) ----
    configs = []
    if args.stream_frames > 0 and not args.quick:
        wl4 = W.config(4, seed=args.seed, n_frames=args.stream_frames)
        mine = sharding.round_robin(wl4.frames, rank, world)
        arm4 = Arm(wl4, mine, local_rank, args.instances, sleepy_e2e)
        arm4.warm(2)
        barrier()
        d_ms, pts4, _, _ = arm4.run_device(2)
        barrier()
        st4, sl4, _ = arm4.run_device_stages(2)
        d_el = max_over_ranks(d_ms * 1e-3)
        e_s, _, _ = arm4.run_e2e(2)
        e_el = max_over_ranks(e_s)
        barrier()
        pts4_all = sum_over_ranks(pts4)
        roof4 = _roofline(arm4, st4, sl4, pts4 / 2 + len(mine), 2)
        configs.append({"config": "cfg4", "workload": wl4.description + f"; a {args.stream_frames}-frame prefix of the "
                        "4096-frame stream, frame i on GPU i mod N, 4 camera heights (4 meshes) on every GPU",
                        "scaling": "strong", "frames_per_step": args.stream_frames,
                        "value": args.stream_frames * 2 / d_el, "unit": "frames/s", "nodes_per_s": pts4_all / d_el,
                        "ms_per_step": 1e3 * d_el / 2,
                        "e2e": {"value": args.stream_frames * 2 / e_el, "unit": "frames/s",
                                "h2d_bytes_per_step": int(sum_over_ranks(sum(arm4.sizes))),
                                "d2h_bytes_per_step": int(sum_over_ranks(arm4.d2h_bytes))},
                        "dominant_kernel": {"kernel": roof4["kernel"], "frac": roof4["frac"],
                                            "achieved_gbs": roof4["achieved"],
                                            "share_of_gpu_time": roof4["share_of_gpu_time"]}})
        arm4.close()
        del arm4
        torch.cuda.empty_cache()

    # ---- one GPU only: parity of every frame of every configuration, the other configurations, the CPU baseline ----
    cpu, parity = None, None
    if rank == 0 and world == 1 and not args.quick:
        import refharness as R
        if not args.no_parity and R.available():
            import parity as P
            parity, detail = {}, {}
            for cfg in range(5):
                rep = P.config_parity(cfg, P.FULL_PARITY_FRAMES[cfg], seed=args.seed)
                parity[f"cfg{cfg}"] = rep["pass"]
                detail[f"cfg{cfg}"] = rep
            parity["detail"] = detail
            parity["tolerances"] = {"pixel_coordinates_px": P.TOL_PX, "classifications_abs": P.TOL_CLS,
                                    "indices": "bit-exact except reported border nodes"}
        if not args.no_other_configs:
            for cfg in (0, 2, 3):
                configs.append(_other_config(cfg, args, local_rank, (parity or {}).get("detail", {}).get(f"cfg{cfg}")))
            if parity and configs and configs[0]["config"] == "cfg4":
                d = parity["detail"]["cfg4"]
                configs[0]["cpu_baseline"] = {"value": d["frames"] / d["reference_seconds"], "unit": "frames/s",
                                              "cores": cores, "kind": "reference",
                                              "sample": f"the {d['frames']} frames of the parity check, one pass"}
        if not args.no_cpu_baseline:
            sample = frames[:min(len(frames), args.cpu_frames)]
            secs, pts, kind, used = _cpu_reference_run(wl, sample, cores)
            cpu = {"value": len(sample) / secs, "unit": "frames/s", "cores": used, "kind": kind,
                   "sample": f"first {len(sample)} frames of the batch, one pass", "nodes_per_s": pts / secs}

    if rank == 0:
        config = _config_block(wl, per_gpu, points / args.steps / per_gpu, world)
        config["result_digest"] = digest
        config["result_digest_of"] = "offsets, pixel_coordinates, global_indices, neighbourhood, classifications of frames 0..63"
        e2e = {"value": e2e_value, "unit": "frames/s", "h2d_bytes_per_step": h2d_bytes * world,
               "d2h_bytes_per_step": d2h_bytes * world, "ms_per_step": 1e3 * e2e_elapsed / args.steps,
               "engine_instances": args.instances,
               "host_waits": "sleeping" if sleepy_e2e else "spinning"}
        if copy_s:
            e2e["copy_bound_ms"] = 1e3 * copy_s
            e2e["frac_of_bound"] = copy_s / (e2e_elapsed / args.steps)
            e2e["copy_bound_note"] = ("the same bytes as bare pinned copies, both directions at once, every rank at the "
                                      "same time, no kernels: the ceiling of this box's host-device path")
        line = {
            "metric": "frames/s", "value": value, "unit": "frames/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": 1e3 * elapsed / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "nodes_per_s": total_points / elapsed, "config": config, "e2e": e2e,
            "gpu_launches": int(launches) * world, "roofline": roofline, "cpu_baseline": cpu, "clocks": clocks,
            "sustained": sustained, "stages": stages, "wall_ms_per_step": 1e3 * wall / args.steps,
            "configs": configs, "parity": parity,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=1)
    ap.add_argument("--frames", type=int, default=64, help="frames per GPU per step")
    ap.add_argument("--cpu-frames", type=int, default=32, help="frames of the bounded CPU sample beside our arm")
    ap.add_argument("--instances", type=int, default=2, help="engine instances (host threads) of the end-to-end arm")
    ap.add_argument("--stream-frames", type=int, default=1024,
                    help="frames of configuration 4's stream that are dealt over the GPUs (0: skip)")
    ap.add_argument("--sustained-seconds", type=float, default=2.5)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--no-other-configs", action="store_true")
    ap.add_argument("--quick", action="store_true", help="the headline's two timed arms only (for profiler captures)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
