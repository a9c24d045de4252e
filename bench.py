#!/usr/bin/env python
"""Benchmark: encrypted matmuls of one BERT-base encoder layer (forward + LoRA backward) on N B200s.

  python bench.py --gpus N --steps K --warmup W        (N > 1: launched with torch.distributed.run)
  python bench.py --impl reference ...                  CPU arm: the oracle port on the host cores

A step is one pass over the layer's matmul units (12 ct x pt groups with 132 fused plaintext products,
42 two-tile ct x ct products = 84 tile products, 18 of them with a transpose).  Units are independent
and are dealt to the ranks by estimated cost; the K-groups of a ct x pt sublayer that land on different ranks
exchange their partial output tiles (point to point, to one owner per tile).  Total work is fixed, so the line
says "strong".  The timed passes replay a CUDA graph of one pass over operands resident in HBM.

Prints one JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import ctypes as C
import importlib
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
PKG = "encryption-friendly_llm_architecture_b200"
METRIC = "HE matmul latency ms (BERT-base layer)"
LIMB = 65536 * 8


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """SM clock and throttle reasons sampled DURING the timed region: NVML reads from a thread of this process
    (two light queries every 250 ms; a looping nvidia-smi process was measured to disturb the timed kernels),
    nvidia-smi only if NVML cannot be loaded."""

    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index):
        self.index, self.sm, self.max, self.reasons, self.proc, self.stop_flag, self.thread = index, [], None, set(), None, threading.Event(), None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(vis.split(",")[self.index]) if vis and all(v.strip().isdigit() for v in vis.split(",")) else self.index
            h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            bits = [(pynvml.nvmlClocksEventReasonHwSlowdown, "hw_slowdown"), (pynvml.nvmlClocksEventReasonHwThermalSlowdown, "hw_thermal_slowdown"),
                    (pynvml.nvmlClocksEventReasonSwThermalSlowdown, "sw_thermal_slowdown"), (pynvml.nvmlClocksEventReasonSwPowerCap, "sw_power_cap")]

            def loop():
                while not self.stop_flag.is_set():
                    try:
                        self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                        r = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                        self.reasons.update(name for bit, name in bits if r & bit)
                    except Exception:
                        pass
                    self.stop_flag.wait(0.25)
            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "500"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            r = [x.strip() for x in line.split(",")]
            if r and r[0].replace(".", "").isdigit():
                self.sm.append(float(r[0]))
            if len(r) > 1 and r[1].replace(".", "").isdigit():
                self.max = max(self.max or 0.0, float(r[1]))
            if len(r) >= 6:
                self.reasons.update(self.NAMES[k] for k in range(4) if r[2 + k].lower().startswith("active"))

    def stop(self):
        self.stop_flag.set()
        if self.thread:
            self.thread.join(timeout=2)
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                pass
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.max, "reasons": sorted(self.reasons), "samples": len(self.sm)}


# ---------------------------------------------------------------------------------------------
# CPU arm: exact operation counts of the layer from a dry run of the oracle's schedules, times
# per-operation timings sampled on the host cores.
# ---------------------------------------------------------------------------------------------
def cpu_layer_estimate(pkg, sample_reps=40):
    # launchers export OMP_NUM_THREADS=1; the CPU arm is meant to use every host core (set before libgomp loads)
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    lib_path = os.path.join(ROOT, "oracle", "_build", "liboracle.so")
    if not os.path.exists(lib_path):
        subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle")])
    layer = importlib.import_module(PKG + ".layer")
    prm = pkg.make_params()
    # 1. counts
    dry = pkg.capi.Lib(lib_path, "orc_", prm)
    dry.dll.orc_set_dry(dry.ctx, 1)
    H = pkg.Hemmer(dry)
    wl = layer.LayerWorkload(H, layer.synthetic(1234))
    dry.dll.orc_stats_clear(dry.ctx)
    wl.step()
    need = dry.dll.orc_stats_dump(dry.ctx, None, 0)
    buf = C.create_string_buffer(need)
    dry.dll.orc_stats_dump(dry.ctx, buf, need)
    counts = {}
    for line in buf.value.decode().splitlines():
        op, lvl, n = line.split()
        counts[(op, int(lvl))] = int(n)
    # 2. sampled timings
    o = pkg.capi.Lib(lib_path, "orc_", prm)
    o.keygen()
    o.gen_rot_keys([1])
    z = np.random.default_rng(0).uniform(-1, 1, o.slots)
    top = o.encrypt(o.encode(z, o.L), 1)
    times = {}
    t_all = time.perf_counter()

    def timed(f):
        f()  # first touch of fresh buffers
        t0 = time.perf_counter()
        for _ in range(sample_reps):
            f()
        return (time.perf_counter() - t0) / sample_reps

    for (op, lvl) in sorted(counts):
        ct = top if lvl == o.L else o.level_down(top, lvl)
        if op == "rotate":
            times[(op, lvl)] = timed(lambda: o.rotate(ct, 1))
        elif op == "relin":
            t3 = o.tensor(ct, ct)
            times[(op, lvl)] = timed(lambda: o.relin(t3))
        elif op == "tensor":
            times[(op, lvl)] = timed(lambda: o.tensor(ct, ct))
        elif op in ("rescale", "rescale3"):
            pt = o.encode(z, lvl)
            src = o.mul_pt_norescale(ct, pt) if op == "rescale" else o.tensor(ct, ct)
            times[(op, lvl)] = timed(lambda: o.rescale(src))
        elif op == "mul_pt":
            pt = o.encode(z, lvl)
            times[(op, lvl)] = timed(lambda: o.mul_pt_norescale(ct, pt))
        elif op == "add":
            times[(op, lvl)] = timed(lambda: o.add(ct, ct))
        elif op == "mult_imag":
            times[(op, lvl)] = timed(lambda: o.mult_imag(ct))
        elif op == "scalar_mul":
            times[(op, lvl)] = timed(lambda: o.mult_int(ct, 12345))
        elif op == "encode":
            times[(op, lvl)] = 0.0   # masks and weights are encoded outside the timed region
        elif op == "encrypt":
            times[(op, lvl)] = 0.0   # inputs are resident when the clock starts
        else:
            times[(op, lvl)] = 0.0
    sample_s = time.perf_counter() - t_all
    total_ms = 1e3 * sum(counts[k] * times[k] for k in counts)
    ops = sum(n for (op, _), n in counts.items() if op not in ("encode", "encrypt"))
    return total_ms, {"ops": ops, "sample_seconds": round(sample_s, 1), "distinct_ops_timed": len(times)}


def run_reference(args):
    pkg = importlib.import_module(PKG)
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    per_step = []
    info = {}
    for i in range(args.warmup + args.steps):
        ms, info = cpu_layer_estimate(pkg)
        if i >= args.warmup:
            per_step.append(ms)
    v = statistics.median(per_step)
    sample = (f"layer time = sum over {info['distinct_ops_timed']} distinct (operation, level) pairs of count x sampled time; counts exact from a dry run of "
              f"the reference-faithful schedules ({info['ops']} homomorphic operations), each pair timed once per step on full-size (N=2^16) operands")
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "ms", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": v,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "u64", "data": "synthetic",
            "config": {"workload": "bert_base_layer_matmuls_fwd_plus_lora_bwd", "ring_degree": 65536, "levels": 12, "tile": 128},
            "cpu_baseline": {"value": v, "unit": "ms", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": v, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def golden_units(schedule):
    """Digests recorded from the CPU oracle for one unit of every kind of the layer (tests/golden/golden.json)."""
    path = os.path.join(ROOT, "tests", "golden", "golden.json")
    if not os.path.exists(path):
        return {}
    return json.load(open(path)).get("layer_units", {}).get(f"schedule{schedule}", {})


def run_gpu(args):
    import hashlib
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = importlib.import_module(PKG)
    layer = importlib.import_module(PKG + ".layer")
    lib = pkg.open_gpu(pkg.make_params(), device=local)
    lib.set_host_threads(max(1, (os.cpu_count() or 1) // int(os.environ.get("LOCAL_WORLD_SIZE", world))))
    lib.keygen()
    H = pkg.open_hemmer(lib)
    H.set_schedule(args.schedule)
    lib.dll.hb_stream.restype = C.c_void_p
    lib.dll.hb_launch_count.restype = C.c_uint64
    lib.dll.hb_algorithmic_bytes.restype = C.c_uint64
    stream = torch.cuda.ExternalStream(lib.dll.hb_stream(lib.ctx), device=torch.device("cuda", local))
    wl = layer.LayerWorkload(H, layer.synthetic(1234), rank=rank, world=world)
    if world > 1:   # communicator for the K-split exchange; the 128-byte id travels over torch.distributed
        ident = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            buf = (C.c_ubyte * 128)()
            assert lib.dll.hb_nccl_unique_id(buf) == 0, "NCCL unavailable"
            ident = torch.tensor(list(buf), dtype=torch.uint8)
        ident = ident.cuda()
        dist.broadcast(ident, 0)
        raw = (C.c_ubyte * 128)(*ident.cpu().tolist())
        comm = C.c_void_p()
        lib._chk(lib.dll.hb_nccl_comm_init(lib.ctx, C.c_int(world), C.c_int(rank), raw, C.byref(comm)))
        wl.comm = comm.value

    def barrier():
        lib.sync()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def gather(obj):
        if world == 1:
            return [obj]
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    def timed_region(fn, steps):
        """(max over ranks, this rank's own) device time of `steps` calls of fn, CUDA events on the library's stream."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            for s in range(steps):
                fn(s)   # result handles are dropped at once, as in the warm-up passes: the pool sees the same allocation pattern
            e1.record(stream)
        lib.sync()
        torch.cuda.synchronize()
        own = e0.elapsed_time(e1)
        ms = own
        if world > 1:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        barrier()
        return ms, own

    # operands resident in HBM before the clock starts
    wl.prepare()
    if args.one_step:  # for `ncu --metrics gpu__time_duration.sum`: a warm-up pass (keys, masks), then one pass
        wl.step_resident()
        lib.sync()
        first = int(lib.dll.hb_launch_count(lib.ctx))
        wl.step_resident()
        lib.sync()
        print(json.dumps({"launches_before_second_pass": first}), flush=True)
        print(json.dumps({"one_step": True, "launches": int(lib.dll.hb_launch_count(lib.ctx))}), flush=True)
        return
    for s in range(args.warmup):
        wl.step_resident()
    lib.sync()
    # correctness of this run: every result against the float64 products (max over the ranks), every result hashed
    # (one digest over all tiles in canonical order: the same at every rank count), and the units whose residues the
    # CPU oracle recorded compared bit for bit
    err, digests = wl.check(with_digests=True)
    err = max(gather(err))
    all_digests = {}
    for d in gather({repr(k): v for k, v in digests.items()}):
        all_digests.update(d)
    canon = [repr(("p",) + k) for k in wl.tile_keys] + [repr(("c", i)) for i, u in enumerate(wl.units) if u[0] == "ccmm"]
    missing = [k for k in canon if k not in all_digests]
    outputs_sha = hashlib.sha256("".join(all_digests.get(k, "-") for k in canon).encode()).hexdigest()
    gold = golden_units(args.schedule)
    hits = 0
    for name, want in gold.items():
        tag = ("p", *name.split("/")[:2], int(name.split("/")[2])) if "/" in name else ("c", wl.unit_index(name))
        hits += int(all_digests.get(repr(tag)) == want)
    bit_exact = f"{hits}/{len(gold)}"

    # the timed pass: a CUDA graph of one resident pass, replayed (`--no-graph`: launched from the host every time)
    graph = graph_out = None
    if not args.no_graph:
        graph, graph_out = wl.record_graph()
        lib.graph_launch(graph)
        lib.sync()
    step_fn = (lambda s: lib.graph_launch(graph)) if graph is not None else (lambda s: wl.step_resident())
    sampler = ClockSampler(local)
    sampler.start()
    l0 = lib.dll.hb_launch_count(lib.ctx)
    a0 = lib.dll.hb_algorithmic_bytes(lib.ctx)
    ms_total, own_total = timed_region(step_fn, args.steps)
    launches = (lib.dll.hb_launch_count(lib.ctx) - l0) // max(args.steps, 1)
    alg_bytes = (lib.dll.hb_algorithmic_bytes(lib.ctx) - a0) // max(args.steps, 1)
    clocks = sampler.stop()
    ms_step = ms_total / args.steps
    per_rank = gather({"ms": own_total / args.steps, "alg_bytes": alg_bytes, "units": len(wl.mine), "launches": launches})
    if graph is not None:   # the replayed pass must leave exactly the bits of an ordinary pass
        replay = wl.output_digests(graph_out)
        eager = wl.output_digests(wl.step_resident())
        assert replay == eager, "graph replay and host-launched pass differ"
    ms_eager = None
    if graph is not None and not args.no_compare:
        ms_eager = timed_region(lambda s: wl.step_resident(), 1)[0]
    # exchange time: one host-launched pass with CUDA events around the K-split exchange (nothing overlaps it: the
    # library runs on one stream, so all of it is exposed)
    comm_ms = 0.0
    before_exchange = None
    if world > 1:
        evs = []
        def hook(phase):
            e = torch.cuda.Event(enable_timing=True)
            e.record(stream)
            evs.append(e)
        wl.on_comm = hook
        barrier()
        e_start = torch.cuda.Event(enable_timing=True)
        e_start.record(stream)
        wl.step_resident()
        lib.sync()
        wl.on_comm = None
        own_comm = sum(evs[k].elapsed_time(evs[k + 1]) for k in range(0, len(evs) - 1, 2))
        t = torch.tensor([own_comm], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        comm_ms = float(t.item())
        # this rank's own work before it meets its peers, and what it consisted of
        mix = {}
        for i in wl.mine:
            k = layer.unit_kind(wl.units[i])
            mix[k] = mix.get(k, 0) + 1
        before_exchange = gather({"ms": round(e_start.elapsed_time(evs[0]), 2), "units": mix})
    # the recorded pass is not replayed again: drop it and hand the pool's idle buffers back, the passes below use other sizes
    pb, iu = C.c_uint64(), C.c_uint64()
    lib.dll.hb_mem_info(lib.ctx, C.byref(pb), C.byref(iu))
    pool_gb = round(pb.value / 2 ** 30, 1)   # what the timed passes of the default schedule hold
    graph = graph_out = None
    gc.collect()
    lib.dll.hb_release_cached(lib.ctx)
    # the same layer with the reference's own rotation sequence (no hoisting), for comparison
    ms_faithful = None
    faithful_exact = None
    if args.schedule != 0 and not args.no_compare:
        H.set_schedule(0)
        wl.step_resident()
        ms_faithful = timed_region(lambda s: wl.step_resident(), 1)[0]
        gold0 = golden_units(0)
        if gold0:
            _, dg0 = wl.check(with_digests=True)
            merged = {}
            for d in gather({repr(k): v for k, v in dg0.items()}):
                merged.update(d)
            ok = 0
            for name, want in gold0.items():
                tag = ("p", *name.split("/")[:2], int(name.split("/")[2])) if "/" in name else ("c", wl.unit_index(name))
                ok += int(merged.get(repr(tag)) == want)
            faithful_exact = f"{ok}/{len(gold0)}"
        H.set_schedule(args.schedule)
        gc.collect()
        lib.dll.hb_release_cached(lib.ctx)

    # end to end: host matrices in, decrypted host results out, every step
    wl.h2d_bytes = wl.d2h_bytes = 0
    wl.step_e2e()
    wl.h2d_bytes = wl.d2h_bytes = 0
    wl.phases_ms = {}
    e2e_steps = max(1, args.steps)
    ms_e2e = timed_region(lambda s: wl.step_e2e(), e2e_steps)[0] / e2e_steps
    e2e_phases = {k: round(v / e2e_steps, 1) for k, v in wl.phases_ms.items()}
    h2d, d2h = wl.h2d_bytes // e2e_steps, wl.d2h_bytes // e2e_steps
    if world > 1:
        t = torch.tensor([h2d, d2h, launches, alg_bytes], device="cuda", dtype=torch.float64)
        dist.all_reduce(t)
        h2d, d2h, launches, alg_bytes = int(t[0].item()), int(t[1].item()), int(t[2].item()), int(t[3].item())

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # roofline of the dominant kernel family (NTT) on a batch, timed alone with CUDA events.  The layer passes leave the
    # pool holding most of the device memory in sizes these probes do not use: hand the idle buffers back first.
    gc.collect()
    lib.dll.hb_release_cached(lib.ctx)
    hbm, which = peaks()
    roof = {}
    nb, lvl = 64, lib.L
    bt = lib.ct_create(lvl, 2, nb)
    for inverse in (False, True):
        for _ in range(3):
            lib.ntt(bt, inverse)
        reps = 10
        ms = timed_single(torch, stream, lib, lambda: lib.ntt(bt, inverse), reps)
        limbs = nb * 2 * (lvl + 1)
        alg = limbs * 2 * LIMB                      # each limb read once and written once
        roof["intt" if inverse else "ntt"] = {"algorithmic_bytes": alg, "ms": ms, "gbs": alg / ms / 1e6}
    del bt
    # key switching: rotation of a batch by one step (automorphism + hybrid key switch)
    lib.gen_rot_keys([1])
    ks = {}
    for lv in (12, 4):
        nbk = 32
        cb = lib.ct_create(lv, 2, nbk)
        for _ in range(2):
            lib.rotate(cb, 1)
        ms = timed_single(torch, stream, lib, lambda: lib.rotate(cb, 1), 5)
        n = lv + 1
        beta = {12: 4, 4: 2}[lv]
        alg = (nbk * 4 * n + 2 * beta * (n + 3)) * LIMB
        ks[f"rotate_l{lv}"] = {"algorithmic_bytes": alg, "ms": ms, "gbs": alg / ms / 1e6, "frac": alg / ms / 1e6 / hbm}
        del cb
    # one wrapped copy of a shift loop (schedule 2) at the level of the layer's product loops: two masked rotations of
    # the batch and one division by P*q_l.  Ciphertexts in (2n) and out (2(n-1)); the two masked keys once per batch.
    lv, nbk = 6, 32
    cb = lib.ct_create(lv, 2, nbk)
    lib.ct_zero(cb)
    lib.gen_rot_keys([1, -127])
    ones = np.ones(lib.slots)
    k1, k2 = lib.masked_key(1, lib.encode_ext(ones, lv)), lib.masked_key(-127, lib.encode_ext(ones, lv))
    dgt = lib.decompose(cb)
    for _ in range(2):
        lib.assemble_masked(cb, dgt, k1, k2)
    ms = timed_single(torch, stream, lib, lambda: lib.assemble_masked(cb, dgt, k1, k2), 5)
    alg = (nbk * (4 * (lv + 1) - 2) + 2 * 2 * 2 * (lv + 4)) * LIMB
    ks["wrapped_copy_l6"] = {"algorithmic_bytes": alg, "ms": ms, "gbs": alg / ms / 1e6, "frac": alg / ms / 1e6 / hbm}
    del cb, dgt, k1, k2
    top = roof["ntt"]
    # Instruction roofline of the same transform: a butterfly on a prime below 2^44 is eight FP64 instructions (exact
    # product and its error term, quotient estimate, remainder, the two outputs), and this GPU issues one FP64 warp
    # instruction per two cycles per SM sub-partition (16 lanes), so the FP64 pipe alone bounds the transform below.
    mhz = clocks.get("sm_mhz") or clocks.get("sm_max_mhz") or 1965.0
    bfly = nb * 2 * (lvl + 1) * (65536 // 2) * 16
    fp64_ms = bfly * 8 / (148 * 4 * 16 * mhz * 1e6) * 1e3
    hbm_ms = NTT_TRAFFIC_FACTOR * top["algorithmic_bytes"] / (hbm * 1e6)
    # two launches (column pass, row pass) make one transform: per-launch algorithmic bytes are half of the transform's
    roofline = {"bound": "hbm", "kernel": NTT_KERNELS, "achieved": top["gbs"], "peak": hbm,
                "unit": "GB/s", "frac": top["gbs"] / hbm, "peak_source": which, "traffic": NTT_TRAFFIC_FACTOR * top["algorithmic_bytes"],
                "traffic_source": NTT_TRAFFIC_NOTE,
                "fp64_pipe_bound_ms": fp64_ms, "hbm_traffic_bound_ms": hbm_ms, "measured_ms": top["ms"],
                "bound_note": "FP64 pipe: butterflies x 8 instructions / (148 SMs x 4 sub-partitions x 16 lanes x sampled SM clock); HBM: both passes' traffic / measured copy bandwidth",
                "intt_gbs": roof["intt"]["gbs"], "keyswitch": ks}

    cpu_ms, info = cpu_layer_estimate(pkg) if world == 1 and not args.no_cpu else (None, {})
    cpu = None
    if cpu_ms is not None:
        cpu = {"value": cpu_ms, "unit": "ms", "cores": os.cpu_count() or 1, "kind": "port",
               "sample": f"sum over {info['distinct_ops_timed']} distinct (operation, level) pairs of exact count x one sampled full-size timing ({info['sample_seconds']} s of CPU work)"}
    line = {"metric": METRIC, "value": ms_step, "unit": "ms", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "u64", "data": "synthetic",
            "config": {"workload": "bert_base_layer_matmuls_fwd_plus_lora_bwd", "units": len(wl.units), "batched_calls": True, "schedule": {0: "reference_sequence", 1: "direct_hoisted", 2: "direct_hoisted_one_division_per_copy"}[args.schedule], "ring_degree": 65536, "levels": 12, "tile": 128,
                       "l2": "working set per step is tens of GB, far above the 126 MB L2", "max_abs_err_vs_float64": err,
                       "bit_exact_units": bit_exact, "bit_exact_units_reference_sequence": faithful_exact, "outputs_sha256": outputs_sha, "outputs_missing": len(missing),
                       "timed_as": "cuda_graph_replay" if graph is not None else "host_launched", "host_launched_ms": ms_eager,
                       "reference_sequence_ms": ms_faithful, "device_pool_gb": pool_gb},
            "schedule_roofline_ms": alg_bytes / (hbm * 1e6), "algorithmic_bytes_per_step": alg_bytes,
            "comm_ms": comm_ms, "exposed_comm_frac": comm_ms / ms_step if ms_step else None,
            "compute_ms_per_rank": {"min": min(p["ms"] for p in per_rank), "max": max(p["ms"] for p in per_rank), "all": [round(p["ms"], 2) for p in per_rank],
                                    "units": [p["units"] for p in per_rank], "host_launched_before_exchange": before_exchange},
            "roofline": roofline, "cpu_baseline": cpu,
            "e2e": {"value": ms_e2e, "unit": "ms", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "phases_ms_rank0": e2e_phases},
            "gpu_launches": launches, "clocks": clocks}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# which kernels the roofline object describes, and how their DRAM traffic relates to the algorithmic bytes
NTT_KERNELS = "ntt16v2_fwd_cols+ntt16v2_fwd_rows (one forward NTT of 64 ciphertexts, level 12)"
NTT_TRAFFIC_FACTOR = 2
NTT_TRAFFIC_NOTE = "ncu dram bytes of a 32-ciphertext capture, scaled by limbs: each of the two passes reads and writes every limb once (profiles/ntt16v2_passes_level12.md)"


def run_sweep(args):
    """Primitive sweep on a batch of 256 independent ciphertexts with uniform residues, levels 12/8/4/1.
    Prints one JSON object: per operation the time, the algorithmic bytes and the fraction of the measured HBM peak."""
    import torch
    pkg = importlib.import_module(PKG)
    torch.cuda.set_device(0)
    lib = pkg.open_gpu(pkg.make_params(), device=0)
    lib.keygen()
    lib.gen_rot_keys([1, 128, 4096])
    lib.dll.hb_stream.restype = C.c_void_p
    stream = torch.cuda.ExternalStream(lib.dll.hb_stream(lib.ctx), device=torch.device("cuda", 0))
    hbm, which = peaks()
    B, K = args.sweep_batch, 3
    out = {"sweep": f"{B} ciphertexts, N=2^16", "peak_gbs": hbm, "peak_source": which, "rows": []}
    rng = np.random.default_rng(5)
    for lv in [int(x) for x in args.sweep_levels.split(",")]:
        n = lv + 1
        beta = (lv + 1) // 4 + 1            # digits in use: limb i belongs to digit (i+1)/4
        data = np.empty((B, 2, n, lib.N), dtype=np.uint64)
        for l in range(n):
            data[:, :, l, :] = rng.integers(0, int(lib.primes[l]), size=(B, 2, lib.N), dtype=np.uint64)
        ct = lib.ct_create(lv, 2, B)
        lib.ct_import(ct, data)
        del data
        pt = lib.encode(rng.uniform(-1, 1, lib.slots), lv)
        key = 2 * beta * (n + K)
        ops = [("ntt", lambda: lib.ntt(ct, False), B * 2 * n * 2), ("intt", lambda: lib.ntt(ct, True), B * 2 * n * 2)]
        for st in (1, 128, 4096):
            ops.append((f"rotate{st}", lambda st=st: lib.rotate(ct, st), B * 4 * n + key))
        ops.append(("tensor+relin", lambda: lib.relin(lib.tensor(ct, ct)), B * 6 * n + key))
        if lv >= 1:
            prod = lib.mul_pt_norescale(ct, pt)
            ops.append(("rescale", lambda: lib.rescale(prod), B * (4 * n - 2)))
        if lv >= 1:
            # one wrapped copy of a shift loop: two masked rotations of the batch + one division by P*q_l.  Reads the
            # ciphertexts (2n), writes them one level down (2(n-1)); the lifted digits are made once per operand and
            # shared by all 127 copies, so they and the two masked keys count once per batch.
            lib.gen_rot_keys([1, -127])
            m = (rng.uniform(0, 1, lib.slots) > 0.5).astype(np.float64)
            k1, k2 = lib.masked_key(1, lib.encode_ext(m, lv)), lib.masked_key(-127, lib.encode_ext(1.0 - m, lv))
            dg = lib.decompose(ct)
            ops.append(("wrapped_copy", lambda: lib.assemble_masked(ct, dg, k1, k2), B * (4 * n - 2) + 2 * key))
        if args.sweep_ops:
            ops = [o for o in ops if o[0] in args.sweep_ops.split(",")]
        for name, fn, limbs in ops:
            fn(); fn()
            ms = timed_single(torch, stream, lib, fn, 3)
            alg = limbs * LIMB
            out["rows"].append({"op": name, "level": lv, "ms": round(ms, 4), "algorithmic_bytes": alg, "gbs": round(alg / ms / 1e6, 1), "frac": round(alg / ms / 1e6 / hbm, 4)})
        del ct, pt, ops
        prod = k1 = k2 = dg = None
        gc.collect()
        lib.dll.hb_release_cached(lib.ctx)  # the next level's buffers have other sizes: do not let the pool run the device out of memory
    print(json.dumps(out), flush=True)


def timed_single(torch, stream, lib, fn, reps):
    lib.sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(reps):
            keep = fn()
        e1.record(stream)
    lib.sync()
    return e0.elapsed_time(e1) / reps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--one-step", action="store_true", help="run a single pass of the layer and exit (launch-list profiling)")
    ap.add_argument("--schedule", type=int, default=2, choices=[0, 1, 2],
                    help="0: the reference's rotation sequence; 1: direct, hoisted rotations (same products, fewer chained key switches); "
                         "2 (default): as 1, each wrapped copy of the shift loops made with one division by P*q_level instead of two ModDowns and a rescale")
    ap.add_argument("--no-compare", action="store_true", help="skip the extra timed passes (host-launched, and the reference's rotation sequence)")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel of the timed passes from the host instead of replaying a CUDA graph")
    ap.add_argument("--sweep-ops", type=str, default="", help="comma-separated subset of the sweep's operations (profiling one kernel family)")
    ap.add_argument("--sweep-batch", type=int, default=256)
    ap.add_argument("--sweep-levels", type=str, default="12,8,4,1")
    ap.add_argument("--sweep", action="store_true", help="primitive sweep on 256 ciphertexts instead of the layer")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.sweep:
        run_sweep(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
