"""Throughput of the Visual Mesh hot path on B200s, with the reference CPU engine timed beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config 1] [--impl ours|reference]

A step is one pass of the hot path (device-side lookup, projection, compaction, neighbour remap, image sampling, all
graph-convolution layers) over one batch of synthetic frames; the default workload is configuration 1: 64 seeded
1280x1024 RGBA frames, Ring6/Sphere mesh at h = 1.2 m, equidistant lens with distortion, 8-layer network. One JSON
line is printed by rank 0:

  value      frames/s over all GPUs with the frames already resident in HBM and results left in HBM
  e2e        frames/s through the C ABI with frames in pinned HOST memory and results copied back to the host
  roofline   the dominant kernel (the 16 -> 16 graph-convolution layer) against the measured HBM bandwidth
  cpu_baseline  the reference CPU engine on this box's host cores, on a bounded sample of the same frames

With N > 1 (launched by torchrun, one rank per GPU) every rank runs the same per-GPU batch on its own frames; frames
are independent, so there is no collective on the data path - only a barrier and a max over ranks around the timing.
`--impl reference` times the reference's own CPU engine (oracle/_ref, the unmodified reference compiled in place) with
one engine instance per host core, the pattern of example/benchmark.cpp:86-101,142.
"""
import argparse
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

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu capture summarised in
# profiles/ (None until captured); scaled to the launch's rows when the capture ran a smaller case.
# DRAM traffic per row of the dominant kernels from their ncu captures (dram__bytes_read + dram__bytes_write over the
# rows of the captured launch); traffic grows in proportion to the rows, so it is scaled to the bench's launches.
NCU_TRAFFIC_BYTES_PER_ROW = {
    (16, 16): 119.6,  # profiles/graph_conv_16x16_cfg1_16frames.md: 132.6 MB over 1,108,261 rows
    (32, 32): 250.4,  # profiles/graph_conv_tc_tmem_32x32_cfg3_1frame.md: 233.3 MB over 931,718 rows
}


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

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

    def stop(self, windows):
        """windows: [(t0, t1)] host-clock intervals of the timed regions. Samples inside them are "under load"; a
        region shorter than the sampling period takes the samples closest to it."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
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
    wl = W.config(args.config, seed=args.seed, n_frames=max(args.cpu_frames, 1))
    cores = os.cpu_count() or 1
    frames = wl.frames[:args.cpu_frames]
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
        "config": {"workload": wl.name + ": " + wl.description, "frames_per_step": len(frames),
                   "note": "reference CPU engine, one fresh engine instance per frame, one worker per host core"},
        "cpu_baseline": {"value": fps, "unit": "frames/s", "cores": used, "kind": kind,
                         "sample": f"{len(frames)} frames of {wl.name} per step"},
        "e2e": {"value": fps, "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------------------------------

def run_ours(args, rank, world, local_rank):
    import torch
    from visualmesh_b200.engine import Engine, FrameInput, Mesh

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU fallback")
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
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(x):
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    sampler = ClockSampler(_physical_device(local_rank))
    sampler.start()
    per_gpu = args.frames
    wl = W.config(args.config, seed=args.seed, n_frames=per_gpu * world)
    frames = sharding.shard(wl.frames, rank, world)  # rank r takes its contiguous slice of the seeded stream
    engine = Engine(wl.network, device=local_rank)
    meshes = {}
    for fr in frames:
        if fr.mesh.key() not in meshes:
            meshes[fr.mesh.key()] = Mesh.from_spec(fr.mesh)

    # frames: once in pinned host memory (the end-to-end arm) and once in HBM (the device-resident arm)
    sizes = [fr.image_bytes for fr in frames]
    starts = np.concatenate([[0], np.cumsum([(s + 255) // 256 * 256 for s in sizes])]).astype(np.int64)
    host = torch.empty(int(starts[-1]), dtype=torch.uint8, pin_memory=True)
    host_np = host.numpy()
    for i, fr in enumerate(frames):
        host_np[starts[i]:starts[i] + sizes[i]] = fr.image()
    dev = host.cuda(non_blocking=False)
    torch.cuda.synchronize()

    host_frames = [FrameInput(meshes[fr.mesh.key()], fr.Hoc, fr.lens, host_np[starts[i]:starts[i] + sizes[i]],
                              fr.format, None) for i, fr in enumerate(frames)]
    dev_frames = [FrameInput(meshes[fr.mesh.key()], fr.Hoc, fr.lens, dev.data_ptr() + int(starts[i]), fr.format, None,
                             image_on_device=True) for i, fr in enumerate(frames)]
    dev_batch = engine.prepare_batch(dev_frames)

    def stage_names():
        """The engine's stage name of every dense layer, in order (graph_conv_<cin>x<cout> for the first layer of a
        group, dense_<cin>x<cout> for the ones that follow it)."""
        names, width = [], 4
        for group in wl.network:
            for i, layer in enumerate(group):
                cout = layer.biases.shape[0]
                names.append(("graph_conv_" if i == 0 else "dense_") + f"{width}x{cout}")
                width = cout
        return names

    # ---- device-resident arm: `value`, per-kernel times for the roofline ----
    warm = max(args.warmup, 3)
    for _ in range(warm):
        engine.run_prepared(dev_batch, results_on_device=True, time_stages=True, raw=True)
    barrier()
    launches0 = engine.launch_count()
    stage_total, stage_launches = {}, {}
    points = 0
    t0, w0 = time.perf_counter(), time.time()
    engine.timer_start()
    for _ in range(args.steps):
        res = engine.run_prepared(dev_batch, results_on_device=True, time_stages=True, raw=True)
        points += int(res.offsets[res.n_frames])
        for name, ms in engine.stage_times():
            stage_total[name] = stage_total.get(name, 0.0) + ms
            stage_launches[name] = stage_launches.get(name, 0) + 1
    device_ms = engine.timer_stop()
    wall, w1 = time.perf_counter() - t0, time.time()
    launches = engine.launch_count() - launches0
    barrier()
    elapsed = max_over_ranks(device_ms * 1e-3)  # CUDA events on the engine's own stream, max over ranks
    total_frames = per_gpu * world * args.steps
    total_points = sum_over_ranks(points)
    value = total_frames / elapsed
    rows_per_step = points / args.steps + per_gpu  # one off-screen row per frame

    # ---- end-to-end arm: pinned host frames in, results back on the host, copies inside the timed region ----
    # `instances` engine instances, one host thread each, split the batch between them and run their steps back to
    # back - the reference's own advice for its GPU engines (readme/inference.md:70-77, example/benchmark.cpp:86-101,
    # :133): while one instance waits for its last copies the other already uploads its next frames.
    n_inst = max(1, min(args.instances, per_gpu))
    engines = [engine] + [Engine(wl.network, device=local_rank) for _ in range(n_inst - 1)]
    parts = [sharding.shard(host_frames, i, n_inst) for i in range(n_inst)]
    batches = [eng.prepare_batch(part) for eng, part in zip(engines, parts)]
    for eng, b in zip(engines, batches):
        for _ in range(warm):
            eng.run_prepared(b, raw=True)
    d2h_parts = [0] * n_inst

    def e2e_worker(i):
        for _ in range(args.steps):
            res = engines[i].run_prepared(batches[i], raw=True)
            n_pts = int(res.offsets[res.n_frames])
            n_rows = n_pts + res.n_frames
            d2h_parts[i] = (n_pts * (8 + 4) + n_rows * 4 * res.n_neighbours + n_rows * 4 * res.n_classes
                            + 4 * res.n_frames)

    barrier()
    e2e_launches0 = sum(eng.launch_count() for eng in engines)
    t1, w2 = time.perf_counter(), time.time()
    engine.timer_start()
    workers = [threading.Thread(target=e2e_worker, args=(i,)) for i in range(n_inst)]
    for w in workers:
        w.start()
    for w in workers:
        w.join()
    e2e_device_ms = engine.timer_stop()
    e2e_wall, w3 = time.perf_counter() - t1, time.time()
    clocks = sampler.stop([(w0, w1), (w2, w3)])
    d2h = sum(d2h_parts)
    # results are complete on the host when the last worker returns: the host clock is the honest one here
    e2e_elapsed = max_over_ranks(max(e2e_device_ms * 1e-3 if n_inst == 1 else 0.0, e2e_wall))
    barrier()
    e2e_value = total_frames / e2e_elapsed
    launches += sum(eng.launch_count() for eng in engines) - e2e_launches0
    for eng in engines[1:]:
        eng.close()

    # ---- roofline of the dominant kernel ----
    gpu_ms_total = sum(stage_total.values())
    conv = {k: v for k, v in stage_total.items() if k.startswith("graph_conv")}
    top = max(conv, key=conv.get)
    peak, peak_kind = _peaks()
    N = wl.n_neighbours
    cin, cout = [int(v) for v in top.split("_")[-1].split("x")]
    layers_with_name = sum(1 for n in stage_names() if n == top)
    bytes_per_row = 4 * cin + 4 * N + 4 * cout  # each array touched once; neighbour re-reads are expected L2 hits
    rows_total = rows_per_step * args.steps * layers_with_name
    top_s = 1e-3 * stage_total[top]
    achieved = bytes_per_row * rows_total / top_s / 1e9
    roofline = {"bound": "hbm", "kernel": f"k_graph_conv<{cin},{cout}>", "achieved": achieved, "peak": peak,
                "unit": "GB/s", "frac": achieved / peak, "peak_source": f"of {peak_kind}",
                "traffic": (NCU_TRAFFIC_BYTES_PER_ROW[(cin, cout)] * rows_total / stage_launches[top])
                if (cin, cout) in NCU_TRAFFIC_BYTES_PER_ROW else None,
                "algorithmic_bytes_per_launch": bytes_per_row * rows_total / stage_launches[top],
                "avg_launch_ms": stage_total[top] / stage_launches[top],
                "fp32_tflops": 2.0 * (N + 1) * cin * cout * rows_total / top_s / 1e12,
                "share_of_gpu_time": stage_total[top] / gpu_ms_total}
    stages = [{"kernel": k, "ms_per_step": v / args.steps, "launches_per_step": stage_launches[k] / args.steps,
               "share": v / gpu_ms_total} for k, v in sorted(stage_total.items(), key=lambda kv: -kv[1])]

    # ---- CPU baseline beside it (rank 0, N = 1 only) ----
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        sample = frames[:min(len(frames), args.cpu_frames)]
        secs, pts, kind, used = _cpu_reference_run(wl, sample, cores)
        cpu = {"value": len(sample) / secs, "unit": "frames/s", "cores": used, "kind": kind,
               "sample": f"first {len(sample)} frames of the batch, one pass", "nodes_per_s": pts / secs}

    if rank == 0:
        line = {
            "metric": "frames/s", "value": value, "unit": "frames/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": 1e3 * elapsed / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "nodes_per_s": total_points / elapsed,
            "config": {"workload": wl.name + ": " + wl.description, "frames_per_gpu_per_step": per_gpu,
                       "on_screen_nodes_per_frame": points / args.steps / per_gpu,
                       "lookup": "device BSP walk", "l2": "inputs_larger_than_l2",
                       "distortion": "k_px = (k1/W^2, k2/W^4)", "parallelism": f"frame-sharded x{world}"},
            "e2e": {"value": e2e_value, "unit": "frames/s", "h2d_bytes_per_step": int(sum(sizes)) * world,
                    "d2h_bytes_per_step": int(d2h) * world, "ms_per_step": 1e3 * e2e_elapsed / args.steps,
                    "engine_instances": n_inst},
            "gpu_launches": int(launches) * world, "roofline": roofline, "cpu_baseline": cpu, "clocks": clocks,
            "stages": stages, "wall_ms_per_step": 1e3 * wall / args.steps,
        }
        print(json.dumps(line), flush=True)
    engine.close()
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
    ap.add_argument("--cpu-frames", type=int, default=32, help="frames of the bounded CPU sample")
    ap.add_argument("--instances", type=int, default=2, help="engine instances (host threads) of the end-to-end arm")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
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
