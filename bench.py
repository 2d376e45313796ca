#!/usr/bin/env python
"""Benchmark of the persistent GRU scan on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c1|c2|c3|c4|c5] [--impl reference]

Every workload is a ``GRULayer`` of this package built from BASELINE.json's description and run
through its public API: ``out, h_T = layer(x, h0)``, ``out.sum().backward()`` -- input projection
on the tensor-core GEMM core, the CUDA scan, the weight gradients.  Default (every N): config 1,
dense fp32 train step at T=64, B=32 per GPU, I=H=512; with N > 1 each rank runs its own batch
(weak scaling) and the weight gradients are all-reduced over NCCL through
``data_parallel.OverlappedReducer`` (hidden-path bucket, then input-path bucket, each on a side
stream as soon as the backward pass has produced it, reduced where the gradients lie as one
coalesced collective; ``--buckets flat``: through a flat copy; ``--no-overlap``: one ``GradBucket``
at the end).  Metric: sequence-steps/s = T*B*N / step time.  Each line also carries a ``c5`` record: config 5 (dense int8 QAT, T=512, H=1024, B=4096 split over the N GPUs),
three timed steps.

One JSON line on stdout (rank 0).  ``--impl reference`` times the reference's own CPU code
(installed unmodified under oracle/_ref by oracle/make_ref.py) on the host cores instead.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

CONFIGS = {
    # name: kind, T, B (per GPU for c1-c4; TOTAL for c5), H, quant, train, extras
    "c1": dict(kind="dense", T=64, B=32, H=512, quant=False, train=True, wbits=32, h0_scale=0.0,
               desc="dense fp32 train step T=64 B=32/GPU I=H=512"),
    "c2": dict(kind="diagonal", T=1024, B=256, H=1024, quant=True, train=False, wbits=32, h0_scale=0.0,
               desc="diagonal int8-hidden forward T=1024 B=256 I=H=1024"),
    "c3": dict(kind="monarch", T=64, B=32, H=512, quant=True, train=True, wbits=32, h0_scale=0.1, nblocks=8,
               desc="block-diagonal (monarch, 8x64x64 per gate) int8-hidden train step T=64 B=32 I=H=512"),
    "c4": dict(kind="butterfly", T=128, B=64, H=1024, quant=False, train=True, wbits=32, h0_scale=0.0,
               desc="butterfly fp32 train step T=128 B=64 I=H=1024"),
    "c5": dict(kind="dense", T=512, B=4096, H=1024, quant=True, train=True, wbits=8, h0_scale=0.0,
               desc="dense int8-weight int8-hidden train step T=512 B=4096 total I=H=1024, batch-sharded"),
}

# DRAM traffic (dram read + write bytes) of ONE launch of the roofline kernel, from the ncu captures
# summarised under profiles/ (the same bench command under ncu; c2 captured at --T 128 and scaled by
# T, since the kernel streams gi/out once per time step).  None where no capture exists.
ROOFLINE_TRAFFIC = {
    "c1": dict(bytes=15.86e6, T=64),
    "c2": dict(bytes=512.6e6, T=128),
    "c3": dict(bytes=13.11e6, T=64),
    "c4": dict(bytes=212.7e6, T=128),
}
# config 5: one launch of the fused forward step at B = 512 rows per GPU (profiles/): 3.15 MB of weight
# codes (independent of B) + 8.98 MB that scale with the rows (gi[t], h_{t-1}, hidden codes)
C5_STEP_TRAFFIC = dict(fixed=3.15e6, per_512_rows=8.98e6)


# ---------------------------------------------------------------------------
# synthetic problem (same generator on every rank, rank-specific data seed)
# ---------------------------------------------------------------------------

def make_params(cfg, seed=0):
    from oracle import gru_scan_oracle as orc      # generator only (shapes/distributions), not on the timed path
    gen = torch.Generator().manual_seed(seed)
    H = cfg["H"]
    kind = cfg["kind"]
    k = H ** -0.5

    def U(*shape, a):
        return (torch.rand(*shape, generator=gen) * 2 - 1) * a

    if cfg is CONFIGS["c2"] or cfg.get("name") == "c2":
        W, bh = U(3, H, a=1.0), torch.zeros(3 * H)
        Wi, bi = U(3 * H, H, a=1 / 32), torch.zeros(3 * H)
    elif cfg.get("name") == "c3":
        W = torch.randn(3, 8, 64, 64, generator=gen) * 64 ** -0.5
        bh, Wi, bi = U(3 * H, a=k), U(3 * H, H, a=k), U(3 * H, a=k)
    elif cfg.get("name") == "c4":
        W = U(3, 1, 10, 512, 2, 2, a=2 ** -0.5)
        bh, Wi, bi = U(3 * H, a=k), U(3 * H, H, a=k), U(3 * H, a=k)
    elif cfg.get("name") == "c5":
        W, bh, Wi, bi = U(3 * H, H, a=1 / 32), U(3 * H, a=1 / 32), U(3 * H, H, a=1 / 32), U(3 * H, a=1 / 32)
    else:
        W, _ = orc.make_weights(kind, H, gen, nblocks=cfg.get("nblocks", 4))
        bh, Wi, bi = U(3 * H, a=k), U(3 * H, H, a=k), U(3 * H, a=k)
    return dict(W=W, bh=bh, Wi=Wi, bi=bi)


for _n, _c in CONFIGS.items():
    _c["name"] = _n


def calibrated_scale(cfg, params):
    """s = max|h| / 127 from an fp32 forward on a separate seeded batch of 8 sequences
    (a short prefix of T keeps this cheap; h is bounded by 1 anyway)."""
    from oracle import gru_scan_oracle as orc
    gen = torch.Generator().manual_seed(1234)
    T = min(cfg["T"], 32)
    x = torch.randn(T, 8, cfg["H"], generator=gen)
    gi = torch.nn.functional.linear(x, params["Wi"], params["bi"])
    out = orc.scan_forward(cfg["kind"], gi, torch.zeros(8, cfg["H"]), params["W"], params["bh"])
    return float(out.abs().max()) / 127.0


def build_layer(pkg, cfg, params, scale, use_triton):
    """``GRULayer`` of ``pkg`` (this package, or the reference's ``gru_qat``) holding ``params``."""
    H = cfg["H"]
    recipe = pkg.QuantRecipe(weight=pkg.QuantizerConfig(bits=cfg["wbits"], axis=0, name="W"),
                             input_act=pkg.QuantizerConfig(bits=32, name="x_id"),
                             hidden=pkg.QuantizerConfig(bits=8 if cfg["quant"] else 32, mode="frozen", name="h"))
    kind = cfg["kind"]
    structure = None
    if kind != "dense":
        structure = pkg.StructureConfig(kind=kind, nblocks=cfg.get("nblocks", 4))
    layer = pkg.GRULayer(H, H, recipe, gate_layout="fused", structure_hidden=structure, use_triton=use_triton)
    cell = layer.cell
    with torch.no_grad():
        for gi_, g in enumerate("rzn"):
            getattr(cell, f"W_i{g}").copy_(params["Wi"][gi_ * H:(gi_ + 1) * H])
            getattr(cell, f"b_i{g}").copy_(params["bi"][gi_ * H:(gi_ + 1) * H])
            getattr(cell, f"b_h{g}").copy_(params["bh"][gi_ * H:(gi_ + 1) * H])
            if kind == "dense":
                getattr(cell, f"W_h{g}").copy_(params["W"][gi_ * H:(gi_ + 1) * H])
            elif kind == "butterfly":
                getattr(cell, f"struct_Wh_{g}").b.twiddle.copy_(params["W"][gi_][None])
            else:
                getattr(cell, f"struct_Wh_{g}").weight.copy_(params["W"][gi_])
    if cfg["quant"]:
        for q in (cell.quant_h_in, cell.quant_h_out):
            q.scale, q.zero_point, q.config.mode = torch.tensor(float(scale)), torch.tensor(0.0), "frozen"
    return layer


# ---------------------------------------------------------------------------
# device arm
# ---------------------------------------------------------------------------

class DeviceWorkload:
    def __init__(self, name, cfg, rank, world, dev, pinned=True, graph=True, overlap=True):
        import gru_triton_b200 as pkg
        from gru_triton_b200.data_parallel import GradBucket, OverlappedReducer, hidden_then_input_buckets
        self.cfg, self.name, self.rank, self.world, self.dev = cfg, name, rank, world, dev
        self.T, self.H = cfg["T"], cfg["H"]
        self.B = cfg["B"] // world if name == "c5" else cfg["B"]
        p = make_params(cfg)
        self.scale = calibrated_scale(cfg, p) if cfg["quant"] else None
        self.quant = ((self.scale, -127, 127), (self.scale, -127, 127)) if cfg["quant"] else None
        self.layer = build_layer(pkg, cfg, p, self.scale, "auto").to(dev)
        assert self.layer.use_triton, "the benchmark times the CUDA scan path"
        self.layer.train(cfg["train"])
        self.raw = {k: v.to(dev) for k, v in p.items()}
        gen = torch.Generator().manual_seed(100 + rank)
        x = torch.randn(self.T, self.B, self.H, generator=gen)
        h0 = torch.randn(self.B, self.H, generator=gen) * cfg["h0_scale"]
        self.x_host = x.pin_memory() if pinned else None
        self.h0_host = h0.pin_memory() if pinned else None
        self.x, self.h0 = x.to(dev), h0.to(dev)
        del x, h0
        # N > 1: the gradients are summed over the ranks.  Default: two buckets (hidden path, input path),
        # each all-reduced on a side stream as soon as the backward pass has produced it; --no-overlap:
        # one bucket after the backward pass.
        self.bucket = self.reducer = None
        if world > 1 and cfg["train"]:
            if overlap:
                self.reducer = OverlappedReducer(hidden_then_input_buckets(self.layer), in_place=not FLAT_BUCKETS)
            else:
                self.bucket = GradBucket(list(self.layer.parameters()))
        # up to about a thousand batch rows per GPU the step is bound by launch and per-step latency
        # (thousands of small dependent kernels): capture the whole step (forward, loss, backward) once
        self.graphed, self.collective_in_graph = None, False
        if graph and (self.B <= 1024 or graph == "all"):
            from gru_triton_b200 import _lib
            from gru_triton_b200.graphed import GraphedStep
            n0 = _lib.launch_count()
            if self.bucket is not None or self.reducer is not None:
                # the gradient all-reduce is a stream operation like the rest: capture it with the step
                try:
                    self.collective_in_graph = True
                    self.graphed = GraphedStep(self._body, [self.x, self.h0], warmup=3)
                except Exception as e:                      # pragma: no cover - depends on the NCCL build
                    print(f"[bench] capturing the all-reduce failed ({type(e).__name__}: {e}); it runs eagerly",
                          file=sys.stderr)
                    self.collective_in_graph = False
                    if self.reducer is not None:            # fall back to one bucket reduced after the replay
                        self.reducer.remove()
                        self.reducer = None
                        self.bucket = GradBucket(list(self.layer.parameters()))
                    torch.cuda.synchronize()
                    n0 = _lib.launch_count()
            if self.graphed is None:
                self.graphed = GraphedStep(self._body, [self.x, self.h0], warmup=3)
            self.graph_launches = (_lib.launch_count() - n0) / 4      # 3 warm-up passes + the captured one
            # the resident inputs ARE the buffers the captured step reads: no copy per replay
            self.x, self.h0 = self.graphed.static_inputs

    # -- one pass of the hot path through the public API -----------------------
    def _body(self, x, h0):
        if not self.cfg["train"]:
            with torch.no_grad():
                return self.layer(x, h0)[0]
        self.layer.zero_grad(set_to_none=True)
        out, _ = self.layer(x, h0)
        loss = out.sum()
        loss.backward()
        if self.reducer is not None:
            self.reducer.finish()                 # buckets already in flight on the side stream: join them
        elif self.bucket is not None and self.collective_in_graph:
            self.bucket.all_reduce_in_place()     # one coalesced NCCL all-reduce over the .grad tensors
        return loss

    def step(self, x, h0):
        r = self.graphed(x, h0) if self.graphed is not None else self._body(x, h0)
        if self.bucket is not None and not self.collective_in_graph:
            self.bucket.all_reduce_in_place()
        return r

    def scan_only_forward(self):
        """The dominant kernel(s) in isolation: the forward scan on resident gi."""
        from gru_triton_b200 import _lib
        P = self.raw
        qi, qo = self.quant if self.quant else (None, None)
        with torch.no_grad():
            if not hasattr(self, "_gi"):
                self._gi = torch.nn.functional.linear(self.x, P["Wi"], P["bi"])
                self._codes = _lib.quantize_rows(P["W"], 8) if self.cfg["wbits"] <= 8 else None
            kw = {}
            if self.cfg["kind"] == "monarch":
                kw["nblocks"] = P["W"].shape[1]
            if self.cfg["kind"] == "butterfly":
                kw["nblocks"], kw["log2_hpad"] = P["W"].shape[1], P["W"].shape[2]
            if self._codes is not None:
                codes, scales, Wq = self._codes
                return _lib.scan_forward("dense", self._gi, self.h0, Wq, P["bh"], qi, qo, codes=codes, scales=scales)[0]
            return _lib.scan_forward(self.cfg["kind"], self._gi, self.h0, P["W"], P["bh"], qi, qo, **kw)[0]

    def units(self):
        return self.T * self.B

    def scan_fwd_bytes(self):
        return 16 * self.H * self.T * self.B      # gi read 12H + out write 4H per sequence-step

    def tensor_path(self):
        return (self.cfg["kind"] == "dense" and self.H % 32 == 0 and self.B >= 128
                and 12 * self.H * ((self.H + 15) // 16) > 200 * 1024)


class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.path = tempfile.mktemp(suffix=".csv")
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(gpu_index), "-lms", "50"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            f = [c.strip() for c in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        os.unlink(self.path)
        # samples under load = the upper half of the observed clocks
        sm_sorted = sorted(sm)
        load = sm_sorted[len(sm_sorted) // 2:] if sm_sorted else []
        return {"sm_mhz": statistics.median(load) if load else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


def timed_loop(fn, steps, warmup, flush, sync_all):
    """W untimed + K timed calls; each timed call has its own CUDA-event pair on the
    current stream and is preceded by an (untimed) L2 flush.  Returns per-step ms list."""
    for _ in range(warmup):
        flush()
        fn()
    sync_all()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b in evs:
        flush()
        a.record()
        fn()
        b.record()
    sync_all()
    return [a.elapsed_time(b) for a, b in evs]


FLAT_BUCKETS = False       # set by --buckets


def load_peaks():
    ppath = os.path.join(REPO, "MEASURED_PEAKS.json")
    return json.load(open(ppath)) if os.path.exists(ppath) else {}


def tensor_roofline(wl, k_ms, scan_launches, peaks):
    """Forward scan of the tensor-core path: T products [B,H] x [H,3H], int8 codes (exact) or bf16
    planes, against the measured sustained bf16 GEMM rate."""
    flops = 2.0 * wl.T * wl.B * wl.H * 3 * wl.H
    peak_tf = float(peaks.get("bf16_tflops_sustained", 1400.0))
    ach = flops / (k_ms * 1e-3) / 1e12
    fused = getattr(wl, "cfg", {}).get("wbits", 32) <= 8 and getattr(wl, "cfg", {}).get("quant", False)
    return {"kernel": ("tc_fwd_step_kernel, one launch per time step" if fused
                       else "tc_gemm_kernel + gate_fwd_kernel, one pair per time step"), "bound": "tensor",
            "achieved": ach, "peak": peak_tf, "unit": "TFLOP/s", "frac": ach / peak_tf,
            "peak_source": "measured (sustained bf16)" if peaks else "fallback",
            "traffic": (C5_STEP_TRAFFIC["fixed"] + C5_STEP_TRAFFIC["per_512_rows"] * wl.B / 512.0) if fused else None,
            "launch_ms": k_ms / max(scan_launches, 1), "per_step_us": k_ms * 1e3 / wl.T,
            "launches_per_call": scan_launches, "algorithmic_flops_per_launch": flops / wl.T,
            "note": "each step is a small product (B x 3H x H) on the serial chain: the fraction of the tensor "
                    "peak is bounded by per-step latency, reported as per_step_us"}


def run_c5_record(dev, rank, world, flush, sync_all, max_over_ranks, peaks):
    """Config 5 at this N: B = 4096 / N rows per GPU, three timed train steps (device-resident
    inputs), the forward scan alone for its tensor-core fraction, and the all-reduce alone."""
    import torch.distributed as dist
    from gru_triton_b200 import _lib
    cfg = CONFIGS["c5"]
    rec = {"workload": cfg["desc"], "B_per_gpu": cfg["B"] // world, "scaling": "strong"}
    try:
        wl = DeviceWorkload("c5", cfg, rank, world, dev, pinned=False)
        n0 = _lib.launch_count()
        ms = max_over_ranks(timed_loop(lambda: wl.step(wl.x, wl.h0), 3, 1, flush, sync_all))
        rec["gpu_launches_per_step"] = (_lib.launch_count() - n0) / 4
        if wl.graphed is not None:
            rec["gpu_launches_per_step"] = wl.graph_launches   # kernels of the library inside one replay of the graph
        rec["ms_per_step"] = sum(ms) / len(ms)
        rec["seq_steps_per_s"] = cfg["T"] * cfg["B"] / (rec["ms_per_step"] * 1e-3)
        # the collective alone (both buckets back to back when the step overlaps them with the backward);
        # it sums in place, so the gradients are garbage afterwards: they are dropped just below
        if wl.reducer is not None:
            bks = wl.reducer.buckets
            nbytes = sum(p.grad.numel() for b in bks for p in b.params if p.grad is not None) * 4
            ar = max_over_ranks(timed_loop(lambda: [(b.all_reduce() if FLAT_BUCKETS else b.all_reduce_in_place()) for b in bks],
                                           5, 2, flush, sync_all))
        elif wl.bucket is not None:
            nbytes = sum(p.grad.numel() for p in wl.bucket.params if p.grad is not None) * 4
            ar = max_over_ranks(timed_loop(wl.bucket.all_reduce_in_place, 5, 2, flush, sync_all))
        else:
            ar = None
        if ar is not None:
            rec["allreduce_ms"] = statistics.median(ar)
            rec["allreduce_bytes"] = nbytes
            rec["allreduce_overlapped_with_backward"] = wl.reducer is not None
        if wl.reducer is not None:
            wl.reducer.remove()
        wl.layer.zero_grad(set_to_none=True)
        torch.cuda.empty_cache()
        n1 = _lib.launch_count()
        ks = max_over_ranks(timed_loop(wl.scan_only_forward, 3, 1, flush, sync_all))
        rec["roofline"] = tensor_roofline(wl, statistics.median(ks), (_lib.launch_count() - n1) / 4, peaks)
        # whole step: 30 H^2 flops per sequence-step (forward, backward and both weight gradients)
        step_flops = 30.0 * cfg["H"] ** 2 * cfg["T"] * (cfg["B"] // world)
        rec["step_tflops_fp32_equivalent"] = step_flops / (rec["ms_per_step"] * 1e-3) / 1e12
        rec["peak_mem_gb"] = torch.cuda.max_memory_allocated(dev) / 1e9
        del wl
    except torch.cuda.OutOfMemoryError as e:
        rec["error"] = f"out of memory: {str(e)[:120]}"
    torch.cuda.empty_cache()
    return rec


def shutdown(world):
    """Leave a multi-rank run: captured graphs that contain a collective must be gone, and every rank
    past its last collective, before the process group is torn down."""
    import torch.distributed as dist
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        # A destroyed process group can wait for ever on a communicator that a captured graph still
        # references; all results are printed, so leave without running destructors.
        os._exit(0)


def run_device(args):
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch multi-GPU runs with torch.distributed.run (one process per GPU)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from gru_triton_b200 import _lib
    cfg = CONFIGS[args.config]
    if args.T or args.B or args.train:
        cfg = CONFIGS[args.config] = dict(cfg, T=args.T or cfg["T"], B=args.B or cfg["B"],
                                          train=cfg["train"] or args.train)
    wl = DeviceWorkload(args.config, cfg, rank, world, dev, graph=args.graph, overlap=args.overlap)
    graph_note = ("the step (forward, loss, backward) is captured once by gru_triton_b200.graphed.GraphedStep and "
                  "replayed; gpu_launches counts the kernels of the library inside one replay"
                  if wl.graphed is not None else "not used")
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def flush():
        flush_buf.zero_()

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor(ms, device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    sampler = ClockSampler(local) if rank == 0 else None

    # ---- (1) kernel-resident: inputs already in HBM ---------------------------------
    n0 = _lib.launch_count()
    ms = timed_loop(lambda: wl.step(wl.x, wl.h0), args.steps, args.warmup, flush, sync_all)
    launches_per_step = (_lib.launch_count() - n0) / (args.steps + args.warmup)
    if wl.graphed is not None:
        launches_per_step = wl.graph_launches        # kernels of the library inside one replay of the graph
    ms = max_over_ranks(ms)
    ms_per_step = sum(ms) / len(ms)

    # ---- (2) end to end: pinned host -> device copy in, loss (or last h) read back -----
    def e2e_step():
        if wl.graphed is not None:
            # straight into the captured step's input buffers: no staging tensor, no device-to-device copy
            x, h0 = wl.graphed.static_inputs
            x.copy_(wl.x_host, non_blocking=True)
            h0.copy_(wl.h0_host, non_blocking=True)
        else:
            x = wl.x_host.to(dev, non_blocking=True)
            h0 = wl.h0_host.to(dev, non_blocking=True)
        r = wl.step(x, h0)
        return (r if r.dim() == 0 else r[-1, 0, 0]).item()

    ms_e2e = timed_loop(e2e_step, args.steps, args.warmup, flush, sync_all)
    ms_e2e = max_over_ranks(ms_e2e)
    e2e_ms = sum(ms_e2e) / len(ms_e2e)

    # ---- (3) the dominant kernel alone (forward scan), for the roofline --------------
    if cfg["train"]:
        wl.layer.zero_grad(set_to_none=True)
    n1 = _lib.launch_count()
    ks = timed_loop(wl.scan_only_forward, max(min(args.steps, 20), 5), 3, flush, sync_all)
    scan_launches = (_lib.launch_count() - n1) / (max(min(args.steps, 20), 5) + 3)
    k_ms = statistics.median(ks)
    clocks = sampler.stop() if sampler else None
    _lib.check_device_status()        # no bounded wait inside a kernel gave up during the timed loops

    peaks = load_peaks()
    c5 = None
    if args.c5 and args.config == "c1" and not (args.T or args.B or args.train):
        h_bytes = wl.x_host.numel() * 4 + wl.h0_host.numel() * 4
        units_main, tensor_main = wl.units(), wl.tensor_path()
        scan_bytes, Tm, Bm, Hm = wl.scan_fwd_bytes(), wl.T, wl.B, wl.H
        del wl
        torch.cuda.empty_cache()
        c5 = run_c5_record(dev, rank, world, flush, sync_all, max_over_ranks, peaks)
    else:
        h_bytes = wl.x_host.numel() * 4 + wl.h0_host.numel() * 4
        units_main, tensor_main = wl.units(), wl.tensor_path()
        scan_bytes, Tm, Bm, Hm = wl.scan_fwd_bytes(), wl.T, wl.B, wl.H

    if rank != 0:
        shutdown(world)
        return

    peak_gbs = float(peaks.get("hbm_gbs", 6650.0))
    achieved = scan_bytes / (k_ms * 1e-3) / 1e9
    if tensor_main:
        class _W:
            T, B, H, cfg = Tm, Bm, Hm, dict(CONFIGS[args.config])
        roofline = tensor_roofline(_W, k_ms, scan_launches, peaks)
    else:
        latency_bound = cfg["kind"] != "diagonal"
        fp32_peak = 148 * 128 * 2 * 1.965e9 / 1e12          # FMA lanes x 2 flops x max SM clock, nominal
        scan_flops = {"dense": 6.0 * Hm * Hm, "monarch": 6.0 * Hm * (Hm // cfg.get("nblocks", 4)),
                      "butterfly": 9.0 * Hm * max(1, (Hm - 1).bit_length()), "diagonal": 40.0 * Hm}[cfg["kind"]] * Tm * Bm
        roofline = {"kernel": {"dense": "block_fwd_kernel", "monarch": "block_fwd_kernel",
                               "diagonal": "diag_fwd_tma_kernel", "butterfly": "bfly_fwd2_kernel"}[cfg["kind"]],
                    "bound": "latency" if latency_bound else "hbm",
                    "achieved": achieved, "peak": peak_gbs, "unit": "GB/s",
                    "frac": achieved / peak_gbs, "peak_source": "measured" if peaks else "fallback",
                    "traffic": (ROOFLINE_TRAFFIC[args.config]["bytes"] * Tm / ROOFLINE_TRAFFIC[args.config]["T"]
                                if args.config in ROOFLINE_TRAFFIC and not args.B else None),
                    "launch_ms": k_ms, "per_step_us": k_ms * 1e3 / Tm,
                    "launches_per_call": scan_launches,
                    "algorithmic_bytes_per_launch": scan_bytes,
                    "fp32_tflops": scan_flops / (k_ms * 1e-3) / 1e12,
                    "fp32_frac_of_nominal_fma_peak": scan_flops / (k_ms * 1e-3) / 1e12 / fp32_peak}
        if latency_bound:
            roofline["note"] = ("a serial chain of T dependent steps inside one launch: DRAM is nearly idle and no "
                                "pipe is saturated (ncu: profiles/); the bound is the latency of one step, reported "
                                "as per_step_us; frac is the HBM fraction, fp32_frac the FMA-pipe fraction")

    units = units_main * world
    line = {
        "metric": "sequence-steps/sec (T*B/s)", "value": units / (ms_per_step * 1e-3), "unit": "seq-steps/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong" if args.config == "c5" else "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(args.config, cfg, Bm, world, bool(args.T or args.B or args.train)),
        "e2e": {"value": units / (e2e_ms * 1e-3), "unit": "seq-steps/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h_bytes, "d2h_bytes_per_step": 4},
        "gpu_launches": int(round(launches_per_step * args.steps)),
        "gpu_launches_per_step": launches_per_step,
        "cuda_graph": graph_note,
        "clocks": clocks,
        "roofline": roofline,
    }
    if world > 1:
        line["collective"] = {"op": "all-reduce (sum) of the weight gradients, NCCL",
                              "buckets": ("two, overlapped with the backward pass" if args.overlap else "one, after the backward pass")
                                         + (", flat copies" if FLAT_BUCKETS else ", coalesced in place"),
                              "NCCL_NVLS_ENABLE": os.environ.get("NCCL_NVLS_ENABLE", "unset")}
    if c5 is not None:
        line["c5"] = c5
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(args.config, budget_s=15.0)
    if args.kinds and world == 1 and args.config == "c1":
        line["kinds"] = kinds_table(dev, flush, sync_all)
    print(json.dumps(line))
    shutdown(world)


def config_dict(name, cfg, B_per_gpu, world, override):
    d = {"workload": f"{name}: {cfg['desc']}", "T": cfg["T"], "B_per_gpu": B_per_gpu, "H": cfg["H"],
         "hidden_kind": cfg["kind"], "int8_hidden": bool(cfg["quant"]), "weight_bits": cfg["wbits"],
         "train_step": bool(cfg["train"]), "parallelism": f"batch-shard x{world}" if world > 1 else "1 GPU",
         "l2": "256 MiB buffer written between timed steps (outside the timed events)"}
    if override:
        d["override"] = "T / B / train changed on the command line: a profiling case, not a result"
    return d


def kinds_table(dev, flush, sync_all):
    """ms/iter of a train step at the headline shape (T=64, B=32, H=512) per hidden kind."""
    out = {}
    cases = [("dense", "c1", CONFIGS["c1"]), ("monarch_nb8_int8h", "c3", CONFIGS["c3"]),
             ("diagonal", "c1", dict(CONFIGS["c1"], kind="diagonal", name="c1k")),
             ("butterfly", "c1", dict(CONFIGS["c1"], kind="butterfly", name="c1k"))]
    for name, cfgname, cfg in cases:
        wl = DeviceWorkload(cfgname, cfg, 0, 1, dev, pinned=False)
        ms = timed_loop(lambda: wl.step(wl.x, wl.h0), 20, 3, flush, sync_all)
        out[name] = {"ms_per_iter": statistics.median(ms), "seq_steps_per_s": wl.units() / (statistics.median(ms) * 1e-3)}
    out["monarch_two_factor_nb8_int8h"] = two_factor_monarch_case(dev, flush, sync_all)
    return out


def two_factor_monarch_case(dev, flush, sync_all):
    """BASELINE config 3 as worded (two 8 x 64 x 64 factors per gate around the Monarch permutation):
    an extension entry point of this package; the reference's API has one factor per gate."""
    from gru_triton_b200 import tc
    from gru_triton_b200.graphed import GraphedStep
    from gru_triton_b200.scan_monarch import gru_scan_monarch2
    cfg = CONFIGS["c3"]
    T, B, H = cfg["T"], cfg["B"], cfg["H"]
    gen = torch.Generator().manual_seed(7)
    p = make_params(cfg)
    s = calibrated_scale(cfg, p)
    q = (s, -127, 127)
    W1 = (torch.randn(3, 8, 64, 64, generator=gen) * 64 ** -0.5).to(dev).requires_grad_(True)
    W2 = (torch.randn(3, 8, 64, 64, generator=gen) * 64 ** -0.5).to(dev).requires_grad_(True)
    Wi, bi, bh = (p[k].to(dev).requires_grad_(True) for k in ("Wi", "bi", "bh"))
    x = torch.randn(T, B, H, generator=gen).to(dev)
    h0 = (torch.randn(B, H, generator=gen) * cfg["h0_scale"]).to(dev)
    params = [W1, W2, Wi, bi, bh]

    def body(x, h0):
        for t in params:
            t.grad = None
        out = gru_scan_monarch2(tc.linear(x, Wi, bi), h0, W1, W2, bh, h_in_quant=q, h_out_quant=q)
        loss = out.sum()
        loss.backward()
        return loss

    step = GraphedStep(body, [x, h0])
    ms = timed_loop(lambda: step(x, h0), 20, 3, flush, sync_all)
    return {"ms_per_iter": statistics.median(ms), "seq_steps_per_s": T * B / (statistics.median(ms) * 1e-3),
            "note": "extension (no reference parity): dense kernels on the materialised P^T B2 P B1"}


# ---------------------------------------------------------------------------
# CPU arm: the reference's own code (oracle/_ref), or the oracle's port where it cannot run
# ---------------------------------------------------------------------------

def cpu_problem(name):
    """Bounded sample of the workload for the CPU: full C1/C3; a batch slice of the others."""
    cfg = CONFIGS[name]
    B = {"c1": 32, "c2": 8, "c3": 32, "c4": 8, "c5": 4}[name]
    T = {"c1": 64, "c2": 256, "c3": 64, "c4": 32, "c5": 64}[name]
    sample = (f"T={T}, B={B} of T={cfg['T']}, B={cfg['B']} (sequences and steps are independent units; "
              "throughput per sequence-step)") if (T, B) != (cfg["T"], cfg["B"]) else "the full workload"
    return cfg, T, B, sample


def reference_package():
    """The unmodified reference package installed by oracle/make_ref.py, or None."""
    ref_dir = os.path.join(REPO, "oracle", "_ref")
    if not os.path.isfile(os.path.join(ref_dir, "gru_qat", "__init__.py")):
        return None
    if ref_dir not in sys.path:
        sys.path.insert(0, ref_dir)
    import gru_qat
    return gru_qat


def cpu_step_fn(name):
    """(step function, units per step, sample text, kind, what) for the CPU arm of config `name`."""
    from oracle import gru_scan_oracle as orc
    cfg, T, B, sample = cpu_problem(name)
    p = make_params(cfg)
    scale = calibrated_scale(cfg, p) if cfg["quant"] else None
    quant = ((scale, -127, 127), (scale, -127, 127)) if cfg["quant"] else None
    gen = torch.Generator().manual_seed(100)
    x = torch.randn(T, B, cfg["H"], generator=gen)
    h0 = torch.randn(B, cfg["H"], generator=gen) * cfg["h0_scale"]
    qi, qo = quant if quant else (None, None)
    ref = reference_package()

    if ref is not None and cfg["kind"] in ("dense", "diagonal"):
        layer = build_layer(ref, cfg, p, scale, False)           # the reference's per-step PyTorch path

        def step():
            if cfg["train"]:
                layer.zero_grad(set_to_none=True)
                out, _ = layer(x, h0)
                out.sum().backward()
            else:
                with torch.no_grad():
                    layer(x, h0)
        return step, T * B, sample, "reference", "gru_qat.GRULayer(use_triton=False) forward" + (
            " + out.sum().backward()" if cfg["train"] else "")

    if ref is not None and cfg["kind"] == "monarch":
        from gru_qat.triton_kernels import scan_monarch as rm   # torch_structured is absent: scan-form functions
        Wi, bi, W, bh = (p[k].clone().requires_grad_(True) for k in ("Wi", "bi", "W", "bh"))

        def step():
            gi = torch.nn.functional.linear(x, Wi, bi)
            out = rm.gru_scan_monarch_forward_pytorch(gi.detach(), h0, W.detach(), bh.detach(), h_in_quant=qi,
                                                      h_out_quant=qo)
            dgi, _, _, _ = rm.gru_scan_monarch_backward_pytorch(gi.detach(), h0, W.detach(), bh.detach(), out,
                                                                torch.ones_like(out), h_in_quant=qi, h_out_quant=qo)
            gi.backward(dgi)
        return step, T * B, sample, "reference", ("gru_qat gru_scan_monarch_forward_pytorch + _backward_pytorch "
                                                  "(its cell needs the absent torch_structured) + F.linear autograd")

    def step():
        orc.layer_train_step(cfg["kind"], x, h0, p["Wi"], p["bi"], p["W"], p["bh"], qi, qo,
                             weight_bits=cfg["wbits"], backward=cfg["train"])
    return step, T * B, sample, "port", "oracle.layer_train_step (the reference has no CPU path for this kind here)"


def cpu_baseline(name, budget_s):
    torch.set_num_threads(os.cpu_count() or 1)
    step, units, sample, kind, what = cpu_step_fn(name)
    step()
    t0 = time.perf_counter()
    n = 0
    while True:
        step()
        n += 1
        if time.perf_counter() - t0 > budget_s or n >= 50:
            break
    dt = (time.perf_counter() - t0) / n
    return {"value": units / dt, "unit": "seq-steps/s", "cores": torch.get_num_threads(), "kind": kind,
            "ms_per_step": dt * 1e3, "sample": f"{sample}; {n} timed passes of {what}"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = CONFIGS[args.config]
    torch.set_num_threads(os.cpu_count() or 1)
    step, units, sample, kind, what = cpu_step_fn(args.config)
    for _ in range(args.warmup):
        step()
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    dt = sum(times) / len(times)
    v = units / dt
    if args.gpus > 1:
        sample = sample.replace("the full workload", f"one rank's shard (1/{args.gpus} of the job; the host's "
                                "throughput does not depend on how many shards it is given)")
    world = args.gpus
    B_per_gpu = cfg["B"] // world if args.config == "c5" else cfg["B"]
    print(json.dumps({
        "impl": "reference", "metric": "sequence-steps/sec (T*B/s)", "value": v, "unit": "seq-steps/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong" if args.config == "c5" else "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": config_dict(args.config, cfg, B_per_gpu, world, False),
        "cpu_baseline": {"value": v, "unit": "seq-steps/s", "cores": torch.get_num_threads(), "kind": kind,
                         "sample": f"{sample}; {what}"},
        "e2e": {"value": v, "unit": "seq-steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="c1", choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--T", type=int, default=0, help="override the sequence length (profiling a smaller case; "
                    "the line then carries config.override and is not a benchmark result)")
    ap.add_argument("--B", type=int, default=0, help="override the batch, as --T")
    ap.add_argument("--train", action="store_true", help="time forward + backward of a forward-only config "
                    "(a profiling case like --T / --B)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-kinds", dest="kinds", action="store_false")
    ap.add_argument("--no-c5", dest="c5", action="store_false", help="skip the config-5 record of the default run")
    ap.add_argument("--no-graph", dest="graph", action="store_false", help="issue the kernels of a step one by one")
    ap.add_argument("--no-overlap", dest="overlap", action="store_false",
                    help="N > 1: one gradient bucket reduced after the backward pass instead of two overlapped ones")
    ap.add_argument("--graph-all", dest="graph", action="store_const", const="all",
                    help="capture the step in a CUDA graph whatever its size (default: small problems only)")
    ap.add_argument("--buckets", choices=["flat", "in-place"], default="in-place",
                    help="N > 1: all-reduce each bucket through a flat copy, or as one coalesced collective over "
                         "the gradient tensors where they lie")
    args = ap.parse_args()
    global FLAT_BUCKETS
    FLAT_BUCKETS = args.buckets == "flat"
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_device(args)


if __name__ == "__main__":
    main()
