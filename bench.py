#!/usr/bin/env python
"""Benchmark of the Fourier-slice hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline workload (one "step" = one pass of the operator over all poses of the batch):
``project_3d_to_2d_forw`` on a box-256 volume (a 128^3 map zero-padded 2x, fftshifted and
rfftn'd to [1,256,256,129] complex64), 10,000 uniform-SO(3) poses with shifts in +-8 px,
128x128 output, cubic interpolation, oversampling 2, radius cutoff 64.  The JSON line also
carries the back-projection workload (50,000 slices of 128x128 with weights into a box-256
volume, linear interpolation) under ``"backproject"``.

``"sharded_backproject"`` holds the sharded workload: 200,000 slices of 400x400 with weights
into box-800 volumes, split over the ranks (strong scaling), the reduce of the partial volumes
overlapped with the scatter of each rank's last chunk.  ``"parity_check"`` objects compare parts
of the timed outputs with the CPU reference after the timed regions.

With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank processes the
same number of poses on its own replica of the volume (weak scaling, no collective on the
projection path); the back-projection step ends with one NCCL reduce of the partial
data+weight volumes onto rank 0.  Other workloads (``--workload``): the autograd step, the
sharded workload alone, a table of all eight operators, the reference's CUDA kernels and its
published benchmark rows, the reduction-rate ceilings and per-call latency.

``--impl reference`` times the reference's own CPU operators (built by
``oracle/build_ref.py`` into ``oracle/_ref``; the C restatement oracle when that build is
absent) on a bounded sample of the same workload, on rank 0 only.

All inputs are seeded synthetic data of the stated shapes and distributions.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for _p in (ROOT, ROOT / "torch-projectors_b200", ROOT / "tests"):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

import torch  # noqa: E402

# ---- workload definitions ---------------------------------------------------------------
PROJ = dict(name="project_3d_to_2d_forw box-256 (128^3 padded 2x), 10000 poses, 128x128 out, cubic, os=2, cutoff=64",
            vol_box=128, pad=2, P=10_000, N=128, interp="cubic", os=2.0, cutoff=64.0, shift=8.0)
BACK = dict(name="backproject_2d_to_3d_forw 50000 slices 128x128 + weights -> box-256 volumes, linear, os=2",
            P=50_000, N=128, interp="linear", os=2.0, shift=8.0)

# Algorithmic (compulsory) bytes per slice: every distinct input element read once, every
# output element written once, plus one zero-fill pass for atomically accumulated outputs.
PROJ_BYTES_PER_SLICE = 128 * 65 * 8 + 44 + (256 * 256 * 129 * 8) / PROJ["P"]                    # 73,367
BACK_BYTES_PER_SLICE = 128 * 65 * 8 + 128 * 65 * 4 + 44 + 2 * (256 * 256 * 129 * 12) / BACK["P"]  # 103,942

# DRAM traffic per slice of the dominant kernels (dram__bytes_read.sum + dram__bytes_write.sum) from
# ncu captures of a smaller launch of the same kernels, scaled by the slices a launch processes
# (traffic grows in proportion to the slices: the volumes are touched the same way by every slice).
PROJ_TRAFFIC_PER_SLICE = (48.87e6 + 105.01e6) / 2048      # profiles/project_forw_3d_cubic_box256_2048poses.md (current kernel)
# back-projection: two captures of the slab-ordered kernel (4,096 and 16,384 slices) give a part that grows with the
# slices and a fixed part (the workspace); the fixed part also holds the zero-fill and the fold of the workspace
# (profiles/backproject_forw_3d_linear_box256_4096slices.md)
BACK_TRAFFIC_PER_SLICE = (2506.4e6 - 730.7e6) / (16384 - 4096)
BACK_TRAFFIC_FIXED = (730.7e6 - 4096 * BACK_TRAFFIC_PER_SLICE) + 135.3e6 + (135.3e6 + 44.2e6)
# The ceilings the kernels actually sit on (from the same summaries): share of the L1TEX data pipe
# the cubic gather keeps busy.
PROJ_L1TEX_DATA_PIPE_FRAC = 0.909


def reduction_ceiling(taps, ms, pattern):
    """The ceiling that binds the scatter kernels: reductions retired per second against the rate a
    microbenchmark of the same access pattern reaches on an L2-resident buffer."""
    rate = taps / (ms * 1e-3) / 1e9
    return {"bound": "reduction request rate (SM L1TEX-to-crossbar port, measured by the probe)", "achieved": rate, "peak": RED_CEILING_GTAPS[pattern], "unit": "G taps/s",
            "frac": rate / RED_CEILING_GTAPS[pattern], "pattern": pattern,
            "peak_source": "python bench.py --workload red_ceiling (profiles/red_ceiling_b200.md)"}


def measured_peak_gbs():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:  # noqa: BLE001
            pass
    return 6650.0, "fallback"


def uniform_rotations(P, gen, device):
    from cases import random_rotations_3d
    return random_rotations_3d(P, gen).reshape(1, P, 3, 3).to(device)


def make_projection_inputs(device, seed):
    gen = torch.Generator().manual_seed(seed)
    b = PROJ["vol_box"]
    vol = torch.randn(b, b, b, generator=gen).to(device)
    half = b * (PROJ["pad"] - 1) // 2
    pad = torch.nn.functional.pad(vol, (half, half) * 3)
    rec = torch.fft.rfftn(torch.fft.fftshift(pad), norm="forward").to(torch.complex64).unsqueeze(0).contiguous()
    rot = uniform_rotations(PROJ["P"], gen, device)
    shifts = ((torch.rand(1, PROJ["P"], 2, generator=gen) * 2 - 1) * PROJ["shift"]).to(device)
    return rec, rot, shifts


def make_backprojection_inputs(device, seed, P):
    from cases import hermitian_dc_column_
    gen = torch.Generator(device=device).manual_seed(seed)
    N, Nh = BACK["N"], BACK["N"] // 2 + 1
    proj = torch.complex(torch.randn(1, P, N, Nh, generator=gen, device=device),
                         torch.randn(1, P, N, Nh, generator=gen, device=device))
    hermitian_dc_column_(proj)
    weights = torch.rand(1, P, N, Nh, generator=gen, device=device)
    cgen = torch.Generator().manual_seed(seed)
    rot = uniform_rotations(P, cgen, device)
    shifts = ((torch.rand(1, P, 2, generator=cgen) * 2 - 1) * BACK["shift"]).to(device)
    return proj, weights, rot, shifts


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        # nvidia-smi numbers physical GPUs and ignores CUDA_VISIBLE_DEVICES: name the device by its
        # own UUID so that the sampled GPU is the one the kernels run on
        self.lines, self.proc = [], None
        try:
            self.gpu = "GPU-" + str(torch.cuda.get_device_properties(index).uuid)
        except Exception:  # noqa: BLE001
            self.gpu = str(index)

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "25"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "gpu": self.gpu}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, power, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[0])); smax.append(float(f[1])); power.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons), "gpu": self.gpu}


def timed_steps(fn, steps, warmup, flush, barrier):
    """W untimed + K timed calls of fn(); each timed call is bracketed by CUDA events on the
    current stream; L2 is flushed (outside the events) before every call.  Returns the list
    of per-step milliseconds."""
    for _ in range(warmup):
        flush()
        fn()
    torch.cuda.synchronize()
    barrier()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b in evs:
        flush()
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    barrier()
    torch.cuda.synchronize()
    return [a.elapsed_time(b) for a, b in evs]


_CPU_INPUTS = {}


def set_all_threads():
    """All host cores this process may use (torch.distributed.run exports OMP_NUM_THREADS=1)."""
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except (AttributeError, RuntimeError):
        pass
    return torch.get_num_threads()


def cpu_model():
    try:
        for ln in open("/proc/cpuinfo"):
            if ln.lower().startswith("model name"):
                return ln.split(":", 1)[1].strip()
    except OSError:
        pass
    import platform
    return platform.processor() or platform.machine()


def _cpu_projector(kind_wanted="reference"):
    """(callable(n_lo, n_hi) -> seconds, kind, cores) for the projection workload on the host."""
    import oracle
    cores = set_all_threads()
    if "proj" not in _CPU_INPUTS:
        _CPU_INPUTS["proj"] = make_projection_inputs("cpu", seed=1)
    rec, rot, shifts = _CPU_INPUTS["proj"]
    if kind_wanted == "reference" and oracle.reference_available():
        kind = "reference"
        f = oracle.reference_ops().project_3d_to_2d_forw
    else:
        from oracle import port
        kind, cores = "port", 1
        f = port.project_3d_to_2d_forw

    def run(lo, hi):
        t0 = time.perf_counter()
        f(rec, rot[:, lo:hi].contiguous(), shifts[:, lo:hi].contiguous(), [PROJ["N"], PROJ["N"]], PROJ["interp"], PROJ["os"], PROJ["cutoff"])
        return time.perf_counter() - t0
    return run, kind, cores


def run_cpu_sample(kind_wanted="reference"):
    """Time the CPU implementation of the projection workload on a bounded sample: as many of
    the 10,000 poses as take about 10 s, or several passes over all of them on a fast host.
    Returns (slices/s, kind, cores, sample description)."""
    run, kind, cores = _cpu_projector(kind_wanted)
    probe = 64 if kind == "reference" else 8
    dt = run(0, probe)                                # also the warm-up
    n = int(min(PROJ["P"], max(probe, probe * 10.0 / max(dt, 1e-3))))   # ~10 s of CPU work
    dt = run(0, n)
    passes = 1
    while n == PROJ["P"] and dt * passes < 8.0 and passes < 6:          # fast host: more passes
        dt = (dt * passes + run(0, n)) / (passes + 1)
        passes += 1
    return (n / dt, kind, cores,
            f"{n} of the {PROJ['P']} poses of the projection workload, {passes} call(s) of {dt:.1f} s wall each")


def _cpu_checker():
    """(operators, kind): the reference's CPU operators where built, else the C restatement."""
    import oracle
    if oracle.reference_available():
        set_all_threads()
        return oracle.reference_ops(), "reference"
    from oracle import port
    return port, "port"


def check_projection_parity(out, rec, rot, shifts, n=64):
    """n poses of the last timed step's output (the first, the last and seeded random ones)
    against the CPU reference on the same inputs; runs after the timed region."""
    from cases import rel_err
    ops, kind = _cpu_checker()
    P = rot.shape[1]
    g = torch.Generator().manual_seed(99)
    pick = torch.unique(torch.cat([torch.tensor([0, P - 1]), torch.randint(0, P, (n - 2,), generator=g)]))
    want = ops.project_3d_to_2d_forw(rec.cpu(), rot[:, pick.to(rot.device)].cpu().contiguous(), shifts[:, pick.to(rot.device)].cpu().contiguous(),
                                     [PROJ["N"], PROJ["N"]], PROJ["interp"], PROJ["os"], PROJ["cutoff"])
    return {"poses": int(pick.numel()), "against": kind, "max_rel_err": rel_err(out[:, pick.to(out.device)], want), "tol": 1e-5}


def check_backprojection_parity(tp, proj, weights, rot, shifts, dev, n=64):
    """The first n slices of the timed workload back-projected alone by the same entry point
    (workspace included) against the CPU reference; runs after the timed region."""
    from cases import rel_err
    ops, kind = _cpu_checker()
    sub = [x[:, :n].contiguous() for x in (proj, weights, rot, shifts)]
    d, w = tp.backproject_2d_to_3d_forw(sub[0], sub[2], weights=sub[1], shifts=sub[3], interpolation=BACK["interp"], oversampling=BACK["os"])
    d_want, w_want = ops.backproject_2d_to_3d_forw(sub[0].cpu(), sub[1].cpu(), sub[2].cpu(), sub[3].cpu(), BACK["interp"], BACK["os"], None)
    return {"slices": n, "against": kind, "max_rel_err_data": rel_err(d, d_want), "max_rel_err_weights": rel_err(w, w_want), "tol": 1e-4}


def headline_config(world):
    return {"workload": PROJ["name"], "poses_per_gpu": PROJ["P"], "parallelism": f"poses sharded over {world} GPU(s), volume replicated",
            "l2": "flushed before every step (256 MiB memset outside the timed events)"}


def reference_arm(args):
    """Time the reference's CPU operators on the host cores; rank 0 only.  W warm-up and exactly K
    timed steps; each step is the same bounded sample of the workload's poses (about a second of
    CPU work), so that the whole run ends within a few minutes whatever K is."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    run, kind, cores = _cpu_projector("reference")
    probe = 64 if kind == "reference" else 8
    run(0, probe)                                     # first call: thread pool, page faults
    dt = run(0, 8 * probe)
    # per step: all 10,000 poses where the host does them in ~2.5 s (small calls run at a lower rate on
    # many-core hosts, which would flatter the GPU), fewer on slow hosts so that the whole run stays within minutes
    budget_s = min(2.5, 200.0 / max(1, args.steps + args.warmup))
    n = int(min(PROJ["P"], max(probe, 8 * probe * budget_s / max(dt, 1e-4))))
    for _ in range(args.warmup):
        run(0, n)
    per_step = [n / run(0, n) for _ in range(args.steps)]
    value = statistics.median(per_step)
    sample = f"each step: the first {n} of the {PROJ['P']} poses of the projection workload ({n / value:.2f} s wall), {kind} CPU operators"
    line = {
        "impl": "reference", "metric": "Fourier slices/sec (project_3d_to_2d_forw, box 256, 2x oversampling)",
        "value": value, "unit": "slices/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * PROJ["P"] / value, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": headline_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "slices/s", "cores": cores, "cpu_model": cpu_model(), "kind": kind, "sample": sample,
                         "note": "runs on the host CPU; ms_per_step is extrapolated to all 10000 poses"},
        "e2e": {"value": value, "unit": "slices/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def profile_case(args):
    """A small, self-terminating run of one kernel for profiler captures: the same volume
    and slice geometry as the benchmark workloads (so footprints exceed L2 together with the
    pose-major tensors) but only --profile-poses poses, two launches."""
    import torch_projectors_b200 as tp
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    P = args.profile_poses
    rec, rot, shifts = make_projection_inputs(dev, seed=1234)
    rot, shifts = rot[:, :P].contiguous(), shifts[:, :P].contiguous()
    kw = dict(interpolation=args.profile_interp or PROJ["interp"], oversampling=PROJ["os"], fourier_radius_cutoff=PROJ["cutoff"])
    if args.profile_case == "autograd_step":
        # box-512 volume (539 MB), 256x256 slices, cubic, all gradients: forward + backward kernels
        gen = torch.Generator(device=dev).manual_seed(6)
        rec5 = torch.complex(torch.randn(1, 512, 512, 257, generator=gen, device=dev), torch.randn(1, 512, 512, 257, generator=gen, device=dev))
        r5 = uniform_rotations(P, torch.Generator().manual_seed(6), dev).requires_grad_(True)
        s5 = ((torch.rand(1, P, 2, generator=gen, device=dev) * 2 - 1) * 10.0).requires_grad_(True)
        g5 = torch.complex(torch.randn(1, P, 256, 129, generator=gen, device=dev), torch.randn(1, P, 256, 129, generator=gen, device=dev))
        for _ in range(2):
            torch.ops.torch_projectors_b200.project_3d_to_2d_forw(rec5, r5, s5, [256, 256], "cubic", 2.0, None)
            torch.ops.torch_projectors_b200.project_3d_to_2d_back(g5, rec5, r5, s5, "cubic", 2.0, None)
        torch.cuda.synchronize()
        print(f"profile case autograd_step: {P} poses of 256x256 on a box-512 volume, 2 forward + 2 backward launches done")
        return
    if args.profile_case == "step_saving":
        # the same step through the pair of kernels the autograd path runs when rotation gradients are wanted
        gen = torch.Generator(device=dev).manual_seed(6)
        rec5 = torch.complex(torch.randn(1, 512, 512, 257, generator=gen, device=dev), torch.randn(1, 512, 512, 257, generator=gen, device=dev))
        r5 = uniform_rotations(P, torch.Generator().manual_seed(6), dev).requires_grad_(True)
        s5 = ((torch.rand(1, P, 2, generator=gen, device=dev) * 2 - 1) * 10.0).requires_grad_(True)
        g5 = torch.complex(torch.randn(1, P, 256, 129, generator=gen, device=dev), torch.randn(1, P, 256, 129, generator=gen, device=dev))
        order = tp.plane_locality_order(r5.detach())
        for _ in range(2):
            out, der = torch.ops.torch_projectors_b200.project_3d_to_2d_forw_saving(rec5, r5, s5, [256, 256], "cubic", 2.0, None, order)
            torch.ops.torch_projectors_b200.project_3d_to_2d_back_saved(g5, out, der, rec5, r5, s5, "cubic", 2.0, None, order, True)
        torch.cuda.synchronize()
        print(f"profile case step_saving: {P} poses of 256x256 on a box-512 volume, 2 forward + 2 backward launches done")
        return
    if args.profile_case == "project_2d":
        # paper-protocol 2D case: 8 box-256 images, P poses each, linear, oversampling 1, shifts
        from cases import random_rotations_2d
        gen = torch.Generator(device=dev).manual_seed(7)
        rec2 = torch.complex(torch.randn(8, 256, 129, generator=gen, device=dev), torch.randn(8, 256, 129, generator=gen, device=dev))
        rot2 = random_rotations_2d(8 * P, torch.Generator().manual_seed(7)).reshape(8, P, 2, 2).to(dev)
        sh2 = torch.randn(8, P, 2, generator=gen, device=dev) * 5.0
        for _ in range(2):
            tp.project_2d_forw(rec2, rot2, sh2, output_shape=(256, 256), interpolation="linear")
        torch.cuda.synchronize()
        print(f"profile case project_2d: 8 x {P} poses of 256x256, linear, 2 launches done")
        return
    if args.profile_case in ("backproject_slab", "accumulate_slab"):
        # 256x256 slices into box-512 volumes (808 MB > L2): the slab-ordered kernel
        gen = torch.Generator(device=dev).manual_seed(5)
        proj = torch.complex(torch.randn(1, P, 256, 129, generator=gen, device=dev), torch.randn(1, P, 256, 129, generator=gen, device=dev))
        weights = torch.rand(1, P, 256, 129, generator=gen, device=dev)
        brot = uniform_rotations(P, torch.Generator().manual_seed(5), dev)
        if args.profile_case == "accumulate_slab":
            # the streaming path of the sharded workload: persistent interleaved accumulator
            from torch_projectors_b200 import sharding
            vols = sharding.PartialVolumes(1, 512, dev)
            for _ in range(2):
                vols.add_(proj, brot, weights, interpolation="linear", oversampling=2.0)
            vols.flush()
            torch.cuda.synchronize()
            print(f"profile case accumulate_slab: {P} slices of 256x256 into the box-512 accumulator, 2 launches + fold done")
            return
        for _ in range(2):
            tp.backproject_2d_to_3d_forw(proj, brot, weights=weights, interpolation="linear", oversampling=2.0)
        torch.cuda.synchronize()
        print(f"profile case backproject_slab: {P} slices of 256x256 into box 512, 2 launches done")
        return
    if args.profile_case in ("backproject_back", "backproject_cubic", "backproject_2d", "prep"):
        interp = args.profile_interp or "cubic"
        if args.profile_case == "prep":
            # the steps either side: pad + fftshift of a 256^3 map to 512^3, and the way back
            from torch_projectors_b200 import prep
            real = torch.randn(1, 256, 256, 256, device=dev)
            for _ in range(2):
                padded = prep._PadShift.apply(real, 3, 512)
                prep._CropUnshift.apply(padded, 3, 256)
            torch.cuda.synchronize()
            print("profile case prep: 256^3 <-> 512^3, 2 launches of each kernel done")
            return
        if args.profile_case == "backproject_2d":
            # 2D back-projection: P slices of 64x33 with weights into one 128x65 reconstruction
            from cases import random_rotations_2d
            gen = torch.Generator(device=dev).manual_seed(8)
            proj2 = torch.complex(torch.randn(1, P, 64, 33, generator=gen, device=dev), torch.randn(1, P, 64, 33, generator=gen, device=dev))
            w2 = torch.rand(1, P, 64, 33, generator=gen, device=dev)
            rot2 = random_rotations_2d(P, torch.Generator().manual_seed(8)).reshape(1, P, 2, 2).to(dev)
            sh2 = torch.randn(1, P, 2, generator=gen, device=dev) * 3.0
            for _ in range(2):
                tp.backproject_2d_forw(proj2, rot2, weights=w2, shifts=sh2, interpolation=interp, oversampling=2.0)
            torch.cuda.synchronize()
            print(f"profile case backproject_2d: {P} slices of 64x33, {interp}, 2 launches done")
            return
        proj, weights, brot, bshifts = make_backprojection_inputs(dev, 4321, P)
        if args.profile_case == "backproject_cubic":
            for _ in range(2):
                tp.backproject_2d_to_3d_forw(proj, brot, weights=weights, shifts=bshifts, interpolation=interp, oversampling=BACK["os"])
        else:
            gd = torch.randn(1, 256, 256, 129, dtype=torch.complex64, device=dev)
            gw = torch.randn(1, 256, 256, 129, device=dev)
            r_g, s_g = brot.clone().requires_grad_(True), bshifts.clone().requires_grad_(True)
            for _ in range(2):
                torch.ops.torch_projectors_b200.backproject_2d_to_3d_back(gd, gw, proj, weights, r_g, s_g, interp, BACK["os"], None)
        torch.cuda.synchronize()
        print(f"profile case {args.profile_case}: {P} slices, {interp}, 2 launches done")
        return
    for _ in range(2):
        if args.profile_case == "project":
            tp.project_3d_to_2d_forw(rec, rot, shifts, output_shape=(PROJ["N"], PROJ["N"]), **kw)
        elif args.profile_case == "project_back":
            g = torch.randn(1, P, PROJ["N"], PROJ["N"] // 2 + 1, dtype=torch.complex64, device=dev)
            torch.ops.torch_projectors_b200.project_3d_to_2d_back(
                g, rec, rot.clone().requires_grad_(True), shifts.clone().requires_grad_(True),
                PROJ["interp"], PROJ["os"], PROJ["cutoff"])
        else:
            proj, weights, brot, bshifts = make_backprojection_inputs(dev, 4321, P)
            tp.backproject_2d_to_3d_forw(proj, brot, weights=weights, shifts=bshifts, interpolation=BACK["interp"], oversampling=BACK["os"])
    torch.cuda.synchronize()
    print(f"profile case {args.profile_case}: {P} poses, 2 launches done")


# ---- additional workloads (not part of the default line) --------------------------------
STEP = dict(name="autograd step of project_3d_to_2d_forw: box-512 volume (256^3 padded 2x), 4096 poses, 256x256 out, cubic, os=2, MSE loss, grads w.r.t. volume, rotations, shifts",
            vol_box=256, P=4096, N=256, shift=10.0)
SHARD = dict(name="sharded backproject_2d_to_3d_forw: 200000 slices of 400x400 + weights -> box-800 volumes, linear, os=2, chunks of 8192, NCCL reduce",
             P_total=200_000, N=400, chunk=8192, shift=12.0)
# op bytes per autograd step (volume read twice, projections written once and their gradient
# read once, gradient volume zero-filled and written): 4.32 GB = 1.055 MB per slice
STEP_BYTES_PER_SLICE = (2 * 512 * 512 * 257 * 8 + 2 * 4096 * 256 * 129 * 8 + 2 * 512 * 512 * 257 * 8) / 4096
SHARD_BYTES_PER_SLICE = 400 * 201 * 8 + 400 * 201 * 4 + 44
SHARD_PIXELS_PER_SLICE = 62_814          # pixels inside the default cutoff of a 400x201 slice that are scattered
BACK_PIXELS_PER_SLICE = 6_426            # the same for a 128x65 slice
# Reduction ceilings measured by `bench.py --workload red_ceiling` on B200 (L2-resident buffer,
# 10^9 reductions per second).
RED_CEILING_GTAPS = {"one random 16-byte slot per lane": 222.5, "lane pairs on adjacent 16-byte slots": 255.6,
                     "lane pairs sharing a 32-byte sector": 257.3, "four lanes on four adjacent 8-byte voxels": 497.0,
                     "one random 8-byte voxel per lane": 222.5, "lane pairs on adjacent 8-byte voxels": 356.6}


def _dist_setup():
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the B200 path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        opts = dist.ProcessGroupNCCL.Options()
        opts.is_high_priority_stream = True      # the reduce of finished slabs overlaps the scatter of later ones
        dist.init_process_group("nccl", device_id=dev, pg_options=opts)
    return dist, rank, world, local_rank, dev


def autograd_step_workload(args):
    """Autograd-step workload (box-512 volume, 4,096 poses): forward + MSE loss + backward, all three gradients; every rank runs
    the same step on its own replica (weak scaling, no collective)."""
    import torch_projectors_b200 as tp
    dist, rank, world, local_rank, dev = _dist_setup()
    gen = torch.Generator().manual_seed(77 + rank)
    b = STEP["vol_box"]
    vol = torch.randn(b, b, b, generator=gen).to(dev)
    pad = torch.nn.functional.pad(vol, (b // 2, b // 2) * 3)
    rec = torch.fft.rfftn(torch.fft.fftshift(pad), norm="forward").to(torch.complex64).unsqueeze(0).contiguous()
    del vol, pad
    rec.requires_grad_(not args.fixed_volume)
    rot = uniform_rotations(STEP["P"], gen, dev).requires_grad_(True)
    shifts = ((torch.rand(1, STEP["P"], 2, generator=gen) * 2 - 1) * STEP["shift"]).to(dev).requires_grad_(True)
    ggen = torch.Generator(device=dev).manual_seed(78 + rank)
    shape = (1, STEP["P"], STEP["N"], STEP["N"] // 2 + 1)
    target = torch.complex(torch.randn(shape, generator=ggen, device=dev), torch.randn(shape, generator=ggen, device=dev))
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    fwd_ev, bwd_ev = [], []
    # the forward pass keeps its pixels' derivatives for the backward pass (3.2 GB here) unless told otherwise
    saving = not args.no_save_derivatives
    tp.set_save_derivatives(saving)

    def step():
        for t in (rec, rot, shifts):
            t.grad = None
        e0, e1, e2, e3 = (torch.cuda.Event(enable_timing=True) for _ in range(4))
        e0.record()
        out = tp.project_3d_to_2d_forw(rec, rot, shifts, output_shape=(STEP["N"], STEP["N"]), interpolation="cubic", oversampling=2.0)
        e1.record()
        diff = out - target
        loss = (diff.real.square() + diff.imag.square()).mean()
        grad_out = diff * (2.0 / diff.numel())          # d loss / d conj(out) in torch's convention
        e2.record()
        out.backward(grad_out)
        e3.record()
        fwd_ev.append((e0, e1)); bwd_ev.append((e2, e3))
        return loss

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local_rank)
    sampler.start()
    ms = timed_steps(step, args.steps, args.warmup, flush_buf.zero_, barrier)
    clocks = sampler.stop()
    ms_per_step = max_over_ranks(sum(ms) / len(ms))
    f = statistics.median([a.elapsed_time(b) for a, b in fwd_ev[args.warmup:]])
    bw = statistics.median([a.elapsed_time(b) for a, b in bwd_ev[args.warmup:]])
    peak, peak_kind = measured_peak_gbs()
    op_ms = max_over_ranks(f + bw)
    achieved = STEP_BYTES_PER_SLICE * STEP["P"] / (op_ms * 1e-3) / 1e9
    if rank == 0:
        print(json.dumps({
            "metric": "Fourier slices/sec (autograd step of project_3d_to_2d_forw, box 512, 2x oversampling)",
            "value": world * STEP["P"] / (ms_per_step * 1e-3), "unit": "slices/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": STEP["name"], "l2": "inputs (539 MB volume, 1.08 GB projections) exceed L2; 256 MiB flush before every step"},
            "kernels_ms": ({"project_forw_saving_kernel<3,cubic>": f, ("project_back_saved_kernel<3,cubic,rot,shift> (+ memsets)" if args.fixed_volume else "project_back_saved_kernel<3,cubic,rot,shift,rec> (+ memsets)"): bw,
                            "loss and its gradient (torch elementwise)": ms_per_step - f - bw} if saving else
                           {"project_forw_kernel<3,cubic>": f, "project_back_kernel<3,cubic,rot,shift> (+ memsets)": bw,
                            "loss and its gradient (torch elementwise)": ms_per_step - f - bw}),
            "saved_derivatives": saving, "fixed_volume": bool(args.fixed_volume),
            "roofline": {"bound": "hbm", "kernel": "project_forw + project_back (op time only)", "achieved": achieved, "peak": peak,
                         "peak_source": peak_kind, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                         "algorithmic_bytes_per_launch": STEP_BYTES_PER_SLICE * STEP["P"], "launch_ms": op_ms},
            "gpu_launches": 2 * (args.steps + args.warmup), "clocks": clocks}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_sharded_backprojection(dist, rank, world, local_rank, dev, total, overlap_tail=True, check_slices=0, slab_groups=0):
    """Sharded back-projection workload: `total` box-400 slices split over the ranks (strong scaling),
    generated on the device per rank seed in chunks of 8192 outside the timed region; CUDA events
    around the accumulate calls, then the final stage: the rank's last chunk(s), scattered slab by
    slab while finished slabs are folded and reduced onto rank 0 (NCCL) on a second stream.
    Returns the result dict (meaningful on rank 0)."""
    import torch_projectors_b200 as tp
    from torch_projectors_b200 import sharding
    lo, hi = sharding.pose_range(total, rank, world)
    N, Nh = SHARD["N"], SHARD["N"] // 2 + 1
    R = tp._abi.rec_boxsize(N, 2.0)
    kw = dict(interpolation="linear", oversampling=2.0)
    vols = sharding.PartialVolumes(1, R, dev, with_weights=True)
    vols.timing = True
    if slab_groups:
        vols.slab_groups = slab_groups
    gen = torch.Generator(device=dev).manual_seed(900 + rank)
    cgen = torch.Generator().manual_seed(900 + rank)
    # the clock sampler starts here: nvidia-smi needs longer to deliver its first sample than the
    # timed region of an 8-GPU run lasts (two chunks and the final stage), so it also sees the warm-up
    sampler = ClockSampler(local_rank)
    sampler.start()
    # untimed warm-up: the first launch of a kernel pays for loading it (tens of ms when eight
    # processes do so at once), and the first collective for its set-up; a few slices through both
    # stages, then the volumes are cleared again
    wp = torch.complex(torch.randn(1, 64, N, Nh, generator=gen, device=dev), torch.randn(1, 64, N, Nh, generator=gen, device=dev))
    wrot = uniform_rotations(64, cgen, dev)
    for _ in range(3):
        vols.add_(wp, wrot, wp.real.abs().contiguous(), None, **kw)
    vols.add_(wp, wrot, wp.real.abs().contiguous(), None, final=True, **kw)
    vols.reduce(dst=0)
    vols.flat.zero_()
    vols._flat_zero = True
    vols._accumulator()                  # clears the accumulator now, outside the timed region
    del wp

    def make_chunk(n):
        proj = torch.complex(torch.randn(1, n, N, Nh, generator=gen, device=dev), torch.randn(1, n, N, Nh, generator=gen, device=dev))
        weights = torch.rand(1, n, N, Nh, generator=gen, device=dev)
        rot = uniform_rotations(n, cgen, dev)
        shifts = ((torch.rand(1, n, 2, generator=cgen) * 2 - 1) * SHARD["shift"]).to(dev)
        return proj, weights, rot, shifts

    spans = [(c0, min(hi, c0 + SHARD["chunk"])) for c0 in range(lo, hi, SHARD["chunk"])]
    n_final = 1
    if overlap_tail and len(spans) >= 2 and spans[-1][1] - spans[-1][0] < SHARD["chunk"] // 2:
        n_final = 2                        # a short last chunk joins the one before it
    if not overlap_tail:
        n_final = 0
    chunk_ms = []
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches = 0
    for c0, c1 in spans[: len(spans) - n_final]:
        proj, weights, rot, shifts = make_chunk(c1 - c0)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        vols.add_(proj, rot, weights, shifts, **kw)
        b.record()
        torch.cuda.synchronize()
        chunk_ms.append(a.elapsed_time(b))
        launches += 1
        del proj, weights
    # the final stage's slices: generated chunk by chunk like the others, then handed over as one tensor
    final = None
    if n_final:
        parts = [make_chunk(c1 - c0) for c0, c1 in spans[len(spans) - n_final:]]
        final = tuple(torch.cat([p[k] for p in parts], dim=1) for k in range(4)) if len(parts) > 1 else parts[0]
        del parts
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    if final is not None:
        vols.add_(final[0], final[2], final[1], final[3], final=True, **kw)
    vols.reduce(dst=0)
    b.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    final_ms = a.elapsed_time(b)
    # the part of the final stage after its last scatter launch has finished: fold + reduce left exposed
    tail_ms = vols.last_scatter_done.elapsed_time(b) if (final is not None and vols.last_scatter_done is not None) else final_ms
    launches += (vols.slab_groups if final is not None else 0) + 1
    scatter_ms = sum(chunk_ms) + (final_ms - tail_ms)
    t = torch.tensor([scatter_ms + tail_ms, scatter_ms, tail_ms], dtype=torch.float64, device=dev)
    rank_ms = [scatter_ms]
    if world > 1:
        gathered = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(gathered, t)
        rank_ms = [float(x[1]) for x in gathered]
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, scatter_ms, tail_ms = float(t[0]), float(t[1]), float(t[2])
    peak, peak_kind = measured_peak_gbs()
    per_rank = hi - lo
    achieved = (SHARD_BYTES_PER_SLICE * per_rank + 2 * vols.flat.numel() * 4) / (total_ms * 1e-3) / 1e9
    taps = per_rank * SHARD_PIXELS_PER_SLICE * 8
    parity = None
    if rank == 0 and check_slices and final is not None:
        parity = check_sharded_parity(final, check_slices, dev)
    return {
        "metric": "Fourier slices/sec (sharded backproject_2d_to_3d_forw, box 400 -> 800, 2x oversampling)",
        "value": total / (total_ms * 1e-3), "unit": "slices/s", "n_gpus": world, "steps": 1, "warmup": 3,
        "ms_per_step": total_ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": SHARD["name"], "total_slices": total, "slices_per_rank": per_rank,
                   "final_stage_slices": (final[0].shape[1] if final is not None else 0),
                   "timing": "per rank: sum of CUDA-event times of the accumulate calls + the final stage (last chunks scattered slab by slab, "
                             "finished slabs folded and reduced on a second stream meanwhile), max over ranks; chunk generation excluded",
                   "l2": "each 8192-slice chunk (7.9 GB) and the 3.1 GB volumes exceed L2"},
        "scatter_ms": scatter_ms, "fold_and_reduce_ms": tail_ms, "scatter_ms_per_rank": rank_ms, "chunk_ms_rank0": chunk_ms,
        "final_stage_ms_rank0": final_ms,
        "roofline": {"bound": "hbm", "kernel": "backproject_slab_kernel<linear,weights,interleaved> (+ fold_interleaved_kernel, NCCL reduce)",
                     "achieved": achieved, "peak": peak, "peak_source": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "launch_ms": total_ms,
                     "secondary": reduction_ceiling(taps, scatter_ms, "lane pairs on adjacent 16-byte slots")},
        "parity_check": parity,
        "gpu_launches": launches, "clocks": clocks}


def check_sharded_parity(final, n, dev):
    """The first n slices of the final stage once more, alone, through the same slab-by-slab path,
    against the CPU reference on the same slices (outside every timed region)."""
    from cases import rel_err
    from torch_projectors_b200 import sharding
    import torch_projectors_b200 as tp
    proj, weights, rot, shifts = (x[:, :n].contiguous() for x in final)
    R = tp._abi.rec_boxsize(SHARD["N"], 2.0)
    vols = sharding.PartialVolumes(1, R, dev, with_weights=True)
    vols.add_(proj, rot, weights, shifts, interpolation="linear", oversampling=2.0, final=True)
    vols.flush()
    torch.cuda.synchronize()
    ops, kind = _cpu_checker()
    d_want, w_want = ops.backproject_2d_to_3d_forw(proj.cpu(), weights.cpu(), rot.cpu(), shifts.cpu(), "linear", 2.0, None)
    return {"slices": n, "against": kind, "max_rel_err_data": rel_err(vols.data, d_want),
            "max_rel_err_weights": rel_err(vols.weights, w_want), "tol": 1e-4}


def sharded_backprojection_workload(args):
    dist, rank, world, local_rank, dev = _dist_setup()
    res = run_sharded_backprojection(dist, rank, world, local_rank, dev, args.total_slices or SHARD["P_total"],
                                     overlap_tail=not args.no_overlap_tail, check_slices=0 if args.skip_cpu else 32,
                                     slab_groups=args.slab_groups)
    if rank == 0:
        print(json.dumps(res), flush=True)
    if world > 1:
        dist.destroy_process_group()


def ops_table_workload(args):
    """Device-resident timing of all eight raw operators (slices/s each), linear and cubic, at the
    sizes of the three small benchmark workloads: 2D ops on a 128x128 reference (64 px padded 2x), 64x64 output;
    3D ops on the box-256 volume, 128x128 slices.  One JSON object, one entry per operator."""
    import torch_projectors_b200 as tp
    dist, rank, world, local_rank, dev = _dist_setup()
    ops = torch.ops.torch_projectors_b200
    gen = torch.Generator().manual_seed(11)
    ggen = torch.Generator(device=dev).manual_seed(11)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = {}

    def cplx(*shape):
        return torch.complex(torch.randn(*shape, generator=ggen, device=dev), torch.randn(*shape, generator=ggen, device=dev))

    def time_op(name, fn, slices):
        ms = timed_steps(fn, args.steps, args.warmup, flush_buf.zero_, lambda: None)
        m = statistics.median(ms)
        rows[name] = {"ms": m, "slices_per_s": slices / (m * 1e-3)}

    # ---- 2D quartet: config 1 geometry (P = 256) and a throughput-sized batch of poses ----
    from cases import random_rotations_2d
    rec2 = torch.fft.rfft2(torch.fft.fftshift(torch.nn.functional.pad(torch.randn(64, 64, generator=gen), (32, 32, 32, 32))),
                           norm="forward").to(torch.complex64).unsqueeze(0).to(dev)
    for P2 in (256, 65536):
        rot2 = random_rotations_2d(P2, gen).reshape(1, P2, 2, 2).to(dev).requires_grad_(True)
        sh2 = ((torch.rand(1, P2, 2, generator=gen) * 2 - 1) * 4).to(dev).requires_grad_(True)
        proj2 = cplx(1, P2, 64, 33)
        w2 = torch.rand(1, P2, 64, 33, generator=ggen, device=dev)
        gd2, gw2 = cplx(1, 128, 65), torch.randn(1, 128, 65, generator=ggen, device=dev)
        for interp in ("linear", "cubic"):
            tag = f"[P={P2},{interp}]"
            time_op("project_2d_forw" + tag, lambda: ops.project_2d_forw(rec2, rot2, sh2, [64, 64], interp, 2.0, None), P2)
            time_op("project_2d_back" + tag, lambda: ops.project_2d_back(proj2, rec2, rot2, sh2, interp, 2.0, None), P2)
            time_op("backproject_2d_forw" + tag, lambda: ops.backproject_2d_forw(proj2, w2, rot2, sh2, interp, 2.0, None), P2)
            time_op("backproject_2d_back" + tag, lambda: ops.backproject_2d_back(gd2, gw2, proj2, w2, rot2, sh2, interp, 2.0, None), P2)
            if P2 == 65536:
                time_op("project_2d_forw_saving" + tag, lambda: ops.project_2d_forw_saving(rec2, rot2, sh2, [64, 64], interp, 2.0, None), P2)
                o2, d2 = ops.project_2d_forw_saving(rec2, rot2, sh2, [64, 64], interp, 2.0, None)
                time_op("project_2d_back_saved" + tag, lambda: ops.project_2d_back_saved(proj2, o2, d2, rec2, rot2, sh2, interp, 2.0, None, True), P2)
                time_op("project_2d_back_saved, fixed reference" + tag,
                        lambda: ops.project_2d_back_saved(proj2, o2, d2, rec2, rot2, sh2, interp, 2.0, None, False), P2)
                del o2, d2
    # ---- 3D quartet on the box-256 volume ----
    rec3, rot3, sh3 = make_projection_inputs(dev, seed=12)
    P3 = 4096
    rot3 = rot3[:, :P3].contiguous().requires_grad_(True)
    sh3 = sh3[:, :P3].contiguous().requires_grad_(True)
    proj3 = cplx(1, P3, 128, 65)
    w3 = torch.rand(1, P3, 128, 65, generator=ggen, device=dev)
    gd3, gw3 = cplx(1, 256, 256, 129), torch.randn(1, 256, 256, 129, generator=ggen, device=dev)
    for interp in ("linear", "cubic"):
        tag = f"[P={P3},{interp}]"
        time_op("project_3d_to_2d_forw" + tag, lambda: ops.project_3d_to_2d_forw(rec3, rot3, sh3, [128, 128], interp, 2.0, None), P3)
        time_op("project_3d_to_2d_back" + tag, lambda: ops.project_3d_to_2d_back(proj3, rec3, rot3, sh3, interp, 2.0, None), P3)
        time_op("backproject_2d_to_3d_forw" + tag, lambda: ops.backproject_2d_to_3d_forw(proj3, w3, rot3, sh3, interp, 2.0, None), P3)
        time_op("backproject_2d_to_3d_back" + tag, lambda: ops.backproject_2d_to_3d_back(gd3, gw3, proj3, w3, rot3, sh3, interp, 2.0, None), P3)
        time_op("project_3d_to_2d_forw_saving" + tag, lambda: ops.project_3d_to_2d_forw_saving(rec3, rot3, sh3, [128, 128], interp, 2.0, None, None), P3)
        o3, d3 = ops.project_3d_to_2d_forw_saving(rec3, rot3, sh3, [128, 128], interp, 2.0, None, None)
        time_op("project_3d_to_2d_back_saved" + tag, lambda: ops.project_3d_to_2d_back_saved(proj3, o3, d3, rec3, rot3, sh3, interp, 2.0, None, None, True), P3)
        time_op("project_3d_to_2d_back_saved, fixed volume" + tag,
                lambda: ops.project_3d_to_2d_back_saved(proj3, o3, d3, rec3, rot3, sh3, interp, 2.0, None, None, False), P3)
        del o3, d3
    if rank == 0:
        print(json.dumps({"metric": "per-operator device time (all gradients requested in the *_back operators)", "unit": "ms / slices/s",
                          "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "data": "synthetic", "dtype": "f32",
                          "config": {"workload": "all eight raw operators, oversampling 2, shifts, weights; 2D: 128x128 reference -> 64x64; 3D: box-256 volume <-> 128x128",
                                     "l2": "256 MiB flush before every call"},
                          "operators": rows}), flush=True)


def reference_cuda_workload(args):
    """Informational: the reference's own CUDA kernels (recompiled for sm_100 with its flags into
    oracle/_ref by `oracle/build_ref.py --cuda`) timed on the same GPU and inputs as the
    headline workloads, next to this package, with the difference between the two results."""
    import oracle
    if not oracle.reference_cuda_available():
        print(json.dumps({"workload": "reference_cuda", "unavailable": "oracle/_ref/torch_projectors_ref_cuda.so not built"}))
        return
    import torch_projectors_b200 as tp
    from cases import rel_err
    ref = oracle.reference_cuda_ops()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = {}

    def both(name, slices, f_ref, f_new, pick):
        r_ms = statistics.median(timed_steps(f_ref, args.steps, args.warmup, flush_buf.zero_, lambda: None))
        n_ms = statistics.median(timed_steps(f_new, args.steps, args.warmup, flush_buf.zero_, lambda: None))
        a, b = pick(f_ref()), pick(f_new())
        rows[name] = {"reference_cuda_ms": r_ms, "b200_ms": n_ms, "speedup": r_ms / n_ms,
                      "reference_cuda_slices_per_s": slices / (r_ms * 1e-3), "b200_slices_per_s": slices / (n_ms * 1e-3),
                      "max_rel_difference": rel_err(b, a)}

    rec, rot, shifts = make_projection_inputs(dev, seed=1234)
    for interp in ("cubic", "linear"):
        both(f"project_3d_to_2d_forw[{interp}, 10000 poses, box 256]", PROJ["P"],
             lambda: ref.project_3d_to_2d_forw(rec, rot, shifts, [128, 128], interp, 2.0, 64.0),
             lambda: torch.ops.torch_projectors_b200.project_3d_to_2d_forw(rec, rot, shifts, [128, 128], interp, 2.0, 64.0),
             lambda o: o)
    Pb = 20_000
    proj, weights, brot, bshifts = make_backprojection_inputs(dev, 4321, Pb)
    for interp in ("linear", "cubic"):
        both(f"backproject_2d_to_3d_forw[{interp}, {Pb} slices, box 256]", Pb,
             lambda: ref.backproject_2d_to_3d_forw(proj, weights, brot, bshifts, interp, 2.0, None),
             lambda: torch.ops.torch_projectors_b200.backproject_2d_to_3d_forw(proj, weights, brot, bshifts, interp, 2.0, None),
             lambda o: o[0])
    Pg = 2048
    g = proj[:, :Pg].contiguous()
    rot_g = rot[:, :Pg].clone().requires_grad_(True)
    sh_g = shifts[:, :Pg].clone().requires_grad_(True)
    both(f"project_3d_to_2d_back[cubic, {Pg} poses, all grads]", Pg,
         lambda: ref.project_3d_to_2d_back(g, rec, rot_g, sh_g, "cubic", 2.0, 64.0),
         lambda: torch.ops.torch_projectors_b200.project_3d_to_2d_back(g, rec, rot_g, sh_g, "cubic", 2.0, 64.0),
         lambda o: o[0])
    print(json.dumps({"metric": "reference CUDA kernels (sm_100 recompile, --use_fast_math) vs this package, same B200, same inputs",
                      "steps": args.steps, "warmup": args.warmup, "data": "synthetic", "rows": rows}), flush=True)


# Published H100 numbers of the reference (10^3 projections/s; paper/results/tables/*.tex there),
# keyed like the rows produced below: (op, box, B, interp) -> (Fwd, Fwd+Bwd), all at P = 2048, os = 1.
PAPER_H100 = {
    ("project_3d_to_2d", 256, 1, "linear"): (929.5, 149.1), ("project_3d_to_2d", 256, 1, "cubic"): (164.6, 23.0),
    ("project_3d_to_2d", 256, 8, "linear"): (1838.2, 164.6),
    ("project_3d_to_2d", 128, 1, "linear"): (3038.7, 556.9), ("project_3d_to_2d", 128, 1, "cubic"): (632.1, 88.5),
    ("project_3d_to_2d", 128, 8, "linear"): (7729.0, None), ("project_3d_to_2d", 128, 8, "cubic"): (1110.4, None),
    ("backproject_2d_to_3d", 256, 1, "linear"): (135.8, 114.8), ("backproject_2d_to_3d", 256, 1, "cubic"): (18.5, 17.1),
    ("backproject_2d_to_3d", 128, 1, "linear"): (570.3, None), ("backproject_2d_to_3d", 128, 1, "cubic"): (72.5, None),
    ("project_2d", 256, 8, "linear"): (3695.1, 266.8),
}


def paper_matrix_workload(args):
    """The rows of the reference's published benchmark tables re-measured with its protocol:
    oversampling 1, no cutoff argument, complex64 randn data, shifts randn*5, P = 2048, 3 warm-up +
    15 timed runs, median of wall-clock times around the Python call with a device synchronise;
    'Fwd+Bwd' adds the autograd backward of sum(|out|^2) with only the data tensor requiring
    gradients (projections and weights for back-projection)."""
    import torch_projectors_b200 as tp
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    from cases import random_rotations_2d
    gen = torch.Generator().manual_seed(42)
    ggen = torch.Generator(device=dev).manual_seed(42)
    P = 2048
    rows = {}

    def cplx(*shape):
        return torch.complex(torch.randn(*shape, generator=ggen, device=dev), torch.randn(*shape, generator=ggen, device=dev))

    def median_rate(fn, slices):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(15):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            fn()
            torch.cuda.synchronize()
            ts.append(time.perf_counter() - t0)
        return slices / statistics.median(ts) / 1e3            # 10^3 projections per second

    for (op, box, B, interp), (h_fwd, h_both) in PAPER_H100.items():
        rot3 = uniform_rotations(P, gen, dev).expand(B, -1, -1, -1).contiguous()
        shifts = (torch.randn(B, P, 2, generator=gen) * 5.0).to(dev)
        if op == "project_3d_to_2d":
            rec = cplx(B, box, box, box // 2 + 1).requires_grad_(True)
            fwd = lambda: tp.project_3d_to_2d_forw(rec, rot3, shifts, output_shape=(box, box), interpolation=interp)  # noqa: E731

            def both():
                rec.grad = None
                (tp.project_3d_to_2d_forw(rec, rot3, shifts, output_shape=(box, box), interpolation=interp).abs() ** 2).sum().backward()
        elif op == "project_2d":
            rec = cplx(B, box, box // 2 + 1).requires_grad_(True)
            rot2 = random_rotations_2d(B * P, gen).reshape(B, P, 2, 2).to(dev)
            fwd = lambda: tp.project_2d_forw(rec, rot2, shifts, output_shape=(box, box), interpolation=interp)  # noqa: E731

            def both():
                rec.grad = None
                (tp.project_2d_forw(rec, rot2, shifts, output_shape=(box, box), interpolation=interp).abs() ** 2).sum().backward()
        else:
            proj = cplx(B, P, box, box // 2 + 1).requires_grad_(True)
            w = torch.rand(B, P, box, box // 2 + 1, generator=ggen, device=dev).requires_grad_(True)
            fwd = lambda: tp.backproject_2d_to_3d_forw(proj, rot3, weights=w, shifts=shifts, interpolation=interp)  # noqa: E731

            def both():
                proj.grad = None
                w.grad = None
                d, wr = tp.backproject_2d_to_3d_forw(proj, rot3, weights=w, shifts=shifts, interpolation=interp)
                ((d.abs() ** 2).sum() + (wr ** 2).sum()).backward()
        with torch.no_grad():
            r_fwd = median_rate(fwd, B * P)
        r_both = median_rate(both, B * P)
        rows[f"{op} box {box} B={B} {interp}"] = {
            "b200_fwd_kproj_s": r_fwd, "b200_fwd_bwd_kproj_s": r_both, "h100_reference_fwd_kproj_s": h_fwd,
            "h100_reference_fwd_bwd_kproj_s": h_both, "fwd_ratio": r_fwd / h_fwd,
            "fwd_bwd_ratio": (r_both / h_both) if h_both else None}
        torch.cuda.empty_cache()
    print(json.dumps({"metric": "10^3 projections/s with the reference paper's protocol (P = 2048, os = 1): this package on B200 vs the reference's published H100 numbers",
                      "data": "synthetic", "dtype": "f32", "rows": rows}), flush=True)


RED_PATTERNS = ["one random 16-byte slot per lane", "lane pairs on adjacent 16-byte slots", "lane pairs sharing a 32-byte sector",
                "four lanes on four adjacent 8-byte voxels", "one random 8-byte voxel per lane", "lane pairs on adjacent 8-byte voxels"]


def red_ceiling_workload(args):
    """The rate at which red.global.add retires for the access patterns of the scatter kernels
    (library probe, b200proj_reduction_rate_probe): on a 32 MiB buffer (L2-resident: the ceiling
    the scatters are measured against) and on a 2 GiB buffer (what is left when the volume is far
    beyond L2).  148 x 32 blocks of 256 lanes, 64 reductions per lane, CUDA events, median."""
    import torch_projectors_b200 as tp
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    blocks, iters = 148 * 32, 64
    taps = blocks * 256 * iters
    rows = {}
    sampler = ClockSampler(0)
    sampler.start()
    for label, nbytes in (("32 MiB (L2-resident)", 32 << 20), ("2 GiB (beyond L2)", 2 << 30)):
        buf = torch.zeros(nbytes // 4, dtype=torch.float32, device=dev)
        for pattern, name in enumerate(RED_PATTERNS):
            ms = statistics.median(timed_steps(lambda: tp._abi.reduction_rate_probe(pattern, buf, blocks, iters),
                                               max(args.steps, 5), args.warmup, lambda: None, lambda: None))
            rows.setdefault(name, {})[label] = {"ms": ms, "g_taps_per_s": taps / (ms * 1e-3) / 1e9}
        del buf
        torch.cuda.empty_cache()
    # the slab-ordered scatter's memory traffic around the same reductions: a window that fits L2 moves
    # through a 3 GiB target (16 reductions per slot while it is resident), 2 bytes per tap streamed
    target = torch.zeros((3 << 30) // 4, dtype=torch.float32, device=dev)
    source = torch.zeros((1 << 30) // 4, dtype=torch.float32, device=dev)
    s_blocks = 16 * (target.numel() // 4) // (256 * iters)
    for window_mib in (32, 64, 96):
        for keep in (False, True):
            ms = statistics.median(timed_steps(lambda: tp._abi.reduction_rate_probe_streaming(target, window_mib << 20, source, s_blocks, iters, keep),
                                               max(args.steps, 5), args.warmup, lambda: None, lambda: None))
            label = f"{window_mib} MiB window moving through 3 GiB, 2 B per tap streamed from 1 GiB" + (", L2 evict-last hint" if keep else "")
            rows.setdefault(RED_PATTERNS[1], {})[label] = {"ms": ms, "g_taps_per_s": s_blocks * 256 * iters / (ms * 1e-3) / 1e9}
    del target, source
    print(json.dumps({"metric": "red.global.add retired per second by access pattern (10^9 taps/s)", "data": "synthetic",
                      "config": {"workload": f"{blocks} blocks x 256 lanes x {iters} reductions to pseudo-random places"},
                      "rows": rows, "clocks": sampler.stop()}), flush=True)


def latency_workload(args):
    """Per-call cost of the smallest benchmark configuration (project_2d_forw, one 128x65 reference,
    256 poses, 64x64 out, linear, oversampling 2): wall clock per call over a long back-to-back loop
    (the device never idles) through the raw operator, through the public function, and replayed
    from a CUDA graph of ten calls; next to it the reference's own CUDA operator when
    oracle/_ref holds it."""
    import oracle
    import torch_projectors_b200 as tp
    from cases import random_rotations_2d
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    gen = torch.Generator().manual_seed(11)
    rec = torch.fft.rfft2(torch.fft.fftshift(torch.nn.functional.pad(torch.randn(64, 64, generator=gen), (32, 32, 32, 32))),
                          norm="forward").to(torch.complex64).unsqueeze(0).to(dev)
    rot = random_rotations_2d(256, gen).reshape(1, 256, 2, 2).to(dev)
    sh = ((torch.rand(1, 256, 2, generator=gen) * 2 - 1) * 4).to(dev)
    ops = torch.ops.torch_projectors_b200

    def per_call_us(fn, n=3000):
        for _ in range(200):
            fn()
        torch.cuda.synchronize()
        best = None
        for _ in range(5):
            t0 = time.perf_counter()
            for _ in range(n):
                fn()
            torch.cuda.synchronize()
            dt = (time.perf_counter() - t0) / n * 1e6
            best = dt if best is None else min(best, dt)
        return best

    rows = {"raw operator (torch.ops)": per_call_us(lambda: ops.project_2d_forw(rec, rot, sh, [64, 64], "linear", 2.0, None)),
            "public function": per_call_us(lambda: tp.project_2d_forw(rec, rot, sh, output_shape=(64, 64), interpolation="linear", oversampling=2.0))}
    r_g = rot.clone().requires_grad_(True)
    rows["public function, rotations require grad (autograd.Function)"] = per_call_us(
        lambda: tp.project_2d_forw(rec, r_g, sh, output_shape=(64, 64), interpolation="linear", oversampling=2.0))
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for _ in range(3):
            ops.project_2d_forw(rec, rot, sh, [64, 64], "linear", 2.0, None)
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(10):
                out = ops.project_2d_forw(rec, rot, sh, [64, 64], "linear", 2.0, None)
    rows["replayed from a CUDA graph of ten calls"] = per_call_us(graph.replay, n=500) / 10
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(1000):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    rows["device time per call (graph replays, CUDA events)"] = a.elapsed_time(b) / 10000 * 1e3
    if oracle.reference_cuda_available():
        ref = oracle.reference_cuda_ops()
        rows["reference CUDA operator (torch.ops.torch_projectors)"] = per_call_us(lambda: ref.project_2d_forw(rec, rot, sh, [64, 64], "linear", 2.0, None))
    print(json.dumps({"metric": "microseconds per call, project_2d_forw with 256 poses of 64x64 (back-to-back calls, wall clock)",
                      "data": "synthetic", "rows": rows}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--skip-cpu", action="store_true", help="omit the CPU-baseline leg")
    ap.add_argument("--skip-backproject", action="store_true")
    ap.add_argument("--natural-order", action="store_true",
                    help="process slices in the order given (switch the plane-locality order of beyond-L2 volumes off), for comparisons")
    ap.add_argument("--profile-case", choices=["project", "backproject", "project_back", "backproject_slab", "accumulate_slab", "autograd_step", "step_saving", "project_2d",
                                               "backproject_back", "backproject_cubic", "backproject_2d", "prep"], default=None,
                    help="run a few launches of one kernel on a reduced pose count (for ncu captures); prints no bench line")
    ap.add_argument("--profile-poses", type=int, default=2048)
    ap.add_argument("--profile-interp", choices=["linear", "cubic"], default=None, help="--profile-case project: interpolation (default: the workload's cubic)")
    ap.add_argument("--workload", choices=["default", "autograd_step", "sharded_backproject", "ops_table", "reference_cuda", "paper_matrix", "red_ceiling", "latency"], default="default",
                    help="default: projection (+ back-projection) headline line; the other two print their own line")
    ap.add_argument("--total-slices", type=int, default=0, help="sharded_backproject: total slices over all ranks (default 200000)")
    ap.add_argument("--no-overlap-tail", action="store_true", help="sharded_backproject: fold and reduce after the last chunk instead of overlapping them with it")
    ap.add_argument("--slab-groups", type=int, default=0, help="sharded_backproject: launches the final stage is cut into (default: the library's 12)")
    ap.add_argument("--fixed-volume", action="store_true", help="autograd_step: the volume needs no gradient (pose refinement against a fixed reference)")
    ap.add_argument("--no-save-derivatives", action="store_true", help="autograd_step: backward pass that gathers the volume again instead of using derivatives kept by the forward pass")
    ap.add_argument("--skip-sharded", action="store_true", help="default workload: leave the sharded box-400 back-projection out (quick runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    if args.natural_order and args.impl != "reference":
        import torch_projectors_b200.ops as _ops
        _ops.set_pose_order_thresholds(1 << 62, 64)
    if args.profile_case:
        profile_case(args)
        return
    if args.impl == "b200" and args.workload == "autograd_step":
        autograd_step_workload(args)
        return
    if args.impl == "b200" and args.workload == "red_ceiling":
        red_ceiling_workload(args)
        return
    if args.impl == "b200" and args.workload == "latency":
        latency_workload(args)
        return
    if args.impl == "b200" and args.workload == "paper_matrix":
        paper_matrix_workload(args)
        return
    if args.impl == "b200" and args.workload == "reference_cuda":
        reference_cuda_workload(args)
        return
    if args.impl == "b200" and args.workload == "ops_table":
        ops_table_workload(args)
        return
    if args.impl == "b200" and args.workload == "sharded_backproject":
        sharded_backprojection_workload(args)
        return

    if args.impl == "reference":
        reference_arm(args)
        return

    dist, rank, world, local_rank, dev = _dist_setup()

    import torch_projectors_b200 as tp
    from torch_projectors_b200 import sharding

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def flush():
        flush_buf.zero_()        # 256 MiB > the 126 MB L2

    peak, peak_kind = measured_peak_gbs()

    # ---- projection: device-resident inputs --------------------------------------------
    rec, rot, shifts = make_projection_inputs(dev, seed=1234 + rank)
    kw = dict(output_shape=(PROJ["N"], PROJ["N"]), interpolation=PROJ["interp"], oversampling=PROJ["os"],
              fourier_radius_cutoff=PROJ["cutoff"])
    out_holder = {}

    def proj_step():
        out_holder["out"] = tp.project_3d_to_2d_forw(rec, rot, shifts, **kw)

    sampler = ClockSampler(local_rank)
    sampler.start()
    ms = timed_steps(proj_step, args.steps, args.warmup, flush, barrier)
    clocks = sampler.stop()
    ms_per_step = max_over_ranks(sum(ms) / len(ms))
    value = world * PROJ["P"] / (ms_per_step * 1e-3)
    kernel_ms = max_over_ranks(statistics.median(ms))       # one kernel launch per step
    achieved = PROJ_BYTES_PER_SLICE * PROJ["P"] / (kernel_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "project_forw_kernel<3,cubic>", "achieved": achieved, "peak": peak,
                "peak_source": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                "traffic": (PROJ_TRAFFIC_PER_SLICE * PROJ["P"]) if PROJ_TRAFFIC_PER_SLICE else None,
                "algorithmic_bytes_per_launch": PROJ_BYTES_PER_SLICE * PROJ["P"], "launch_ms": kernel_ms,
                "secondary": {"bound": "L1TEX data pipe (64 taps x 8 B per pixel, volume L2-resident)",
                              "frac": PROJ_L1TEX_DATA_PIPE_FRAC, "unit": "l1tex__data_pipe_lsu_wavefronts, fraction of peak",
                              "gather_taps_per_s": 6490 * 64 * PROJ["P"] / (kernel_ms * 1e-3),
                              "peak_source": "ncu capture, profiles/project_forw_3d_cubic_box256_2048poses.md"}}
    parity = None
    if rank == 0 and not args.skip_cpu:
        parity = check_projection_parity(out_holder["out"], rec, rot, shifts)

    # ---- projection end to end: pinned host inputs in, projections back to the host ----
    h_rec = rec.cpu().pin_memory()
    h_rot = rot.cpu().pin_memory()
    h_sh = shifts.cpu().pin_memory()
    h_out = torch.empty((1, PROJ["P"], PROJ["N"], PROJ["N"] // 2 + 1), dtype=torch.complex64).pin_memory()

    def e2e_step():
        # the package's host-to-host call: inputs copied in, chunks of projections copied out on a
        # second stream while the next chunk is computed
        tp.project_3d_to_2d_to_host(h_rec, h_rot, h_sh, out=h_out, chunk=1000, device=dev, **kw)

    e2e_ms = timed_steps(e2e_step, max(3, args.steps // 2), 3, flush, barrier)
    e2e_ms_per_step = max_over_ranks(sum(e2e_ms) / len(e2e_ms))
    h2d = h_rec.numel() * 8 + h_rot.numel() * 4 + h_sh.numel() * 4
    d2h = h_out.numel() * 8
    e2e = {"value": world * PROJ["P"] / (e2e_ms_per_step * 1e-3), "unit": "slices/s", "ms_per_step": e2e_ms_per_step,
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "pcie_gbs": (h2d + d2h) / (e2e_ms_per_step * 1e-3) / 1e9,
           # the value is the mean over the timed steps; the spread shows whether the shared host interfered
           "ms_per_step_median": statistics.median(e2e_ms), "ms_per_step_max": max(e2e_ms)}
    # the same with packed output: only the pixels inside the cutoff leave the device
    n_inside = tp._abi.cutoff_pack_index(PROJ["N"], PROJ["cutoff"], dev)[1]
    h_packed = torch.empty((1, PROJ["P"], n_inside), dtype=torch.complex64).pin_memory()

    def e2e_packed_step():
        tp.project_3d_to_2d_to_host(h_rec, h_rot, h_sh, out=h_packed, chunk=1000, device=dev, packed=True, **kw)

    p_ms = timed_steps(e2e_packed_step, max(3, args.steps // 2), 3, flush, barrier)
    p_ms_per_step = max_over_ranks(sum(p_ms) / len(p_ms))
    e2e_packed = {"value": world * PROJ["P"] / (p_ms_per_step * 1e-3), "unit": "slices/s", "ms_per_step": p_ms_per_step,
                  "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": h_packed.numel() * 8,
                  "pcie_gbs": (h2d + h_packed.numel() * 8) / (p_ms_per_step * 1e-3) / 1e9,
                  "note": f"{n_inside} of {PROJ['N'] * (PROJ['N'] // 2 + 1)} pixels per slice lie inside the cutoff and are copied"}
    del h_packed
    # kernels of this package launched so far: one per device-resident step, one per 1000-pose
    # chunk in every end-to-end step (warm-ups included)
    e2e_chunks = (PROJ["P"] + 999) // 1000
    launches = args.steps + args.warmup + (len(e2e_ms) + 3) * e2e_chunks + (len(p_ms) + 3) * e2e_chunks
    del h_out, out_holder
    torch.cuda.empty_cache()

    # ---- back-projection ----------------------------------------------------------------
    back = None
    if not args.skip_backproject:
        proj, weights, brot, bshifts = make_backprojection_inputs(dev, 4321 + rank, BACK["P"])
        R = tp._abi.rec_boxsize(BACK["N"], BACK["os"])
        vols = sharding.PartialVolumes(1, R, dev, with_weights=True)
        ws_bytes = tp._abi.backproject_workspace_bytes(3, 1, R, BACK["P"], BACK["N"], tp._abi.LINEAR, True)
        workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=dev) if ws_bytes else None
        scatter_ev = []
        back_kernel_name = ("memset(workspace) + backproject_forw_interleaved_kernel<3,linear> + fold_interleaved_kernel" if workspace is not None
                            else "memset(volumes) + backproject_forw_kernel<3,linear,weights>")

        def back_step():
            # zero-fill + scatter (one library call), then the cross-rank reduce when N > 1
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            tp._abi.backproject_forw(3, proj, weights, brot, bshifts, tp._abi.LINEAR, BACK["os"], BACK["N"] / 2.0,
                                     vols.data, vols.weights, False, workspace)
            b.record()
            scatter_ev.append((a, b))
            vols.reduce(dst=0)

        bms = timed_steps(back_step, args.steps, args.warmup, flush, barrier)
        bms_per_step = max_over_ranks(sum(bms) / len(bms))
        scat = max_over_ranks(statistics.median([a.elapsed_time(b) for a, b in scatter_ev[args.warmup:]]))
        bach = BACK_BYTES_PER_SLICE * BACK["P"] / (scat * 1e-3) / 1e9
        back = {"metric": "Fourier slices/sec (backproject_2d_to_3d_forw, box 256, 2x oversampling)",
                "value": world * BACK["P"] / (bms_per_step * 1e-3), "unit": "slices/s", "ms_per_step": bms_per_step,
                "config": {"workload": BACK["name"], "collective": "NCCL reduce of data+weight partial volumes to rank 0" if world > 1 else "none"},
                "roofline": {"bound": "hbm", "kernel": back_kernel_name, "achieved": bach,
                             "peak": peak, "peak_source": peak_kind, "unit": "GB/s", "frac": bach / peak,
                             "traffic": (BACK_TRAFFIC_FIXED + BACK_TRAFFIC_PER_SLICE * BACK["P"]) if workspace is not None else None,
                             "algorithmic_bytes_per_launch": BACK_BYTES_PER_SLICE * BACK["P"], "launch_ms": scat,
                             "secondary": reduction_ceiling(BACK["P"] * BACK_PIXELS_PER_SLICE * 8, scat,
                                                            "lane pairs on adjacent 16-byte slots" if workspace is not None else "lane pairs on adjacent 8-byte voxels")}}
        if rank == 0 and not args.skip_cpu:
            back["parity_check"] = check_backprojection_parity(tp, proj, weights, brot, bshifts, dev)
        launches += (args.steps + args.warmup) * (2 if workspace is not None else 1)     # scatter (+ fold)
        del proj, weights
        torch.cuda.empty_cache()

    # ---- sharded back-projection (box 400 -> 800, strong scaling over the ranks) ---------
    sharded = None
    if not args.skip_sharded:
        sharded = run_sharded_backprojection(dist, rank, world, local_rank, dev, args.total_slices or SHARD["P_total"],
                                             check_slices=0 if args.skip_cpu else 32)
        launches += sharded["gpu_launches"]
        torch.cuda.empty_cache()

    # ---- CPU baseline (rank 0, single-GPU runs only) ------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu:
        v, kind, cores, sample = run_cpu_sample("reference")
        cpu = {"value": v, "unit": "slices/s", "cores": cores, "cpu_model": cpu_model(), "kind": kind, "sample": sample}

    if rank == 0:
        line = {
            "metric": "Fourier slices/sec (project_3d_to_2d_forw, box 256, 2x oversampling)",
            "value": value, "unit": "slices/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": headline_config(world),
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "e2e_packed": e2e_packed, "gpu_launches": launches, "clocks": clocks,
            "parity_check": parity, "backproject": back, "sharded_backproject": sharded,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
