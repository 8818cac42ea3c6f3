#!/usr/bin/env python
"""Benchmark of the denoise hot path on B200.

Metric (BASELINE.json): action chunks/s and p50 chunk latency of the denoise loop.

Default workload ("pi0", BASELINE.json configs[4]): the whole pi0-shaped flow-matching denoise loop --
18 expert layers, hidden 1024, 8 q / 1 kv heads of 256, MLP 4096, prefix of 816 cached K/V rows per layer,
a 50 x 32 action chunk plus the state token, 10 Euler steps -- over 1024 independent observations split
across the ranks (1024 / 512 / 256 / 128 per GPU at 1 / 2 / 4 / 8 GPUs: strong scaling, no collective on the
data path, every rank holds a weight replica and its own K/V pages).  One bench "step" denoises every
observation once, i.e. produces 1024 action chunks.

  python bench.py --gpus N --steps K --warmup W            # this library
  python bench.py --impl reference ...                     # the CPU restatement of the same loop on host cores

At one GPU the same JSON line also carries: the loop's stage timings with the dominant GEMM's roofline, the
pi0 attention kernel against both HBM and tensor peaks, batch-1 / batch-64 chunk latency (configs[2]), and
sub-records for the isolated denoise-attention op (configs[1]), the ternary GEMM sweep and the BitVLA LM stack
(configs[3]) with the reference's own CUDA kernels timed beside them.  --workload selects one of those alone.
"""
import argparse
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

CFG = dict(L=16, T=10, H=720, n_q=15, n_kv=5, hd=64, S=51, P=177, eps=1e-5)
ATTN_BYTES_PER_OBS_LAYER_STEP = 2 * (177 * 5 * 64 * 2) + 2 * (51 * 5 * 64 * 2) + 2 * (51 * 15 * 64 * 2)  # 487,680
# DRAM bytes (read + write) of one attn_hd64_kernel launch per observation, from an ncu capture at batch 64
# (25.11 MB for 64 observations; pages are read once, so the traffic grows in proportion to the batch)
ATTN_DRAM_BYTES_PER_OBS_NCU = 25.11e6 / 64
# int8 tensor-core peak measured on this pool (cuBLASLt 8192^3 through torch._int_mm, best of 10): `--int8-peak`
# repeats the measurement, and the default run measures it again beside the ternary sweep
INT8_PEAK_TOPS = 3249.8


def measure_int8_peak(torch, dev, n=8192):
    """cuBLASLt int8 x int8 -> int32 GEMM (library call, used only as the roofline's denominator)."""
    a = torch.randint(-127, 127, (n, n), dtype=torch.int8, device=dev)
    b = torch.randint(-127, 127, (n, n), dtype=torch.int8, device=dev).t().contiguous().t()
    for _ in range(3):
        torch._int_mm(a, b)
    torch.cuda.synchronize()
    best = 1e9
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        torch._int_mm(a, b)
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(100):
        torch._int_mm(a, b)
    e1.record()
    torch.cuda.synchronize()
    return {"n": n, "burst_tops": 2.0 * n ** 3 / best / 1e9, "sustained_tops": 2.0 * n ** 3 * 100 / e0.elapsed_time(e1) / 1e9,
            "how": "torch._int_mm (cuBLASLt), best of 10 / 100 back to back, CUDA events"}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            t_up = time.monotonic()  # nvidia-smi takes a moment to start: wait for its first line
            while not self.rows and time.monotonic() - t_up < 3.0:
                time.sleep(0.01)
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.monotonic(), [c.strip() for c in line.split(",")]))

    def mark_begin(self):
        """Start of the timed region (the sampler itself is started before the warm-up so that nvidia-smi is up)."""
        self.t0 = time.monotonic()

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        t1 = time.monotonic()
        self.proc.terminate()
        self.thread.join(timeout=2)
        t0 = getattr(self, "t0", 0.0)
        inside = [r for t, r in self.rows if t0 <= t <= t1 + 0.05]
        window = "timed region"
        if not inside:  # region shorter than the sampling interval: the warm-up runs the same load
            inside, window = [r for _, r in self.rows[-3:]], "warm-up (timed region shorter than the sampling interval)"
        sm, mx, reasons = [], None, set()
        for r in inside:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm), "window": window}


def oracle_chunk(orc, rng, n_chunks):
    """CPU restatement of the isolated denoise-attention op for `n_chunks` observations; returns seconds.
    Every input (hidden states included) is generated before the clock starts."""
    c = CFG
    n_rows = (c["n_q"] + 2 * c["n_kv"]) * c["hd"]
    w = orc.bf16_round((rng.standard_normal((c["L"], n_rows, c["H"])) * 0.02).astype(np.float32))
    ln = np.ones(c["H"], np.float32)
    pos = np.arange(c["P"], c["P"] + c["S"]).astype(np.int32)
    kp = rng.standard_normal((c["L"], c["P"], c["n_kv"], c["hd"])).astype(np.float32)
    vp = rng.standard_normal((c["L"], c["P"], c["n_kv"], c["hd"])).astype(np.float32)
    xs = rng.standard_normal((n_chunks, c["T"], c["L"], c["S"], c["H"]), dtype=np.float32)
    kfull = np.concatenate([kp, np.zeros((c["L"], c["S"], c["n_kv"], c["hd"]), np.float32)], axis=1)
    vfull = kfull.copy()
    vfull[:, :c["P"]] = vp
    t0 = time.perf_counter()
    for i in range(n_chunks):
        for step in range(c["T"]):
            for l in range(c["L"]):
                q, k, v = orc.qkv_rope(xs[i, step, l], ln, w[l], pos, c["n_q"], c["n_kv"], c["hd"], c["eps"])
                kfull[l, c["P"]:], vfull[l, c["P"]:] = k, v  # the KV append of the step
                orc.attention(q, kfull[l], vfull[l], c["P"], orc.MASK_SMOLVLA)
    return time.perf_counter() - t0


class OraclePolicyLoop:
    """The CPU restatement (oracle.DenoiseModel) of a whole denoise loop with weights N(0, 0.02), one
    observation per call: the timed CPU baseline of the default workload."""

    def __init__(self, orc, policy, seed):
        c, P = POLICIES[policy]
        rng = np.random.default_rng(seed)
        L, H, I, hd = c["n_layers"], c["H"], c["inter"], c["head_dim"]
        qf, kvf = c["n_q"] * hd, c["n_kv"] * hd
        w = lambda *shape: orc.bf16_round(rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02))
        z = lambda n: np.zeros(n, np.float32)
        one = lambda n: np.ones(n, np.float32)
        cross = [c["model"] == 1 and c["self_every"] > 1 and l % c["self_every"] != 0 for l in range(L)]
        wqkv = []
        for l in range(L):
            kv_in = kvf if cross[l] else H
            wqkv.append(np.concatenate([w(qf, H).ravel(), w(kvf, kv_in).ravel(), w(kvf, kv_in).ravel()]))
        ow = dict(ln_in=[one(H) for _ in range(L)], Wqkv=wqkv, Wo=[w(H, qf) for _ in range(L)],
                  ln_post=[one(H) for _ in range(L)], Wgate=[w(I, H) for _ in range(L)], Wup=[w(I, H) for _ in range(L)],
                  Wdown=[w(H, I) for _ in range(L)], W_sp=w(H, 32) if c["model"] == 0 else None,
                  b_sp=z(H) if c["model"] == 0 else None, W_ain=w(H, 32), b_ain=z(H), W_at1=w(H, 2 * H), b_at1=z(H),
                  W_at2=w(H, H), b_at2=z(H), out_norm=one(H), W_aout=w(32, H), b_aout=z(32))
        ocfg = dict(model=c["model"], n_layers=L, H=H, n_q=c["n_q"], n_kv=c["n_kv"], hd=hd, inter=I, P=P,
                    chunk=c["chunk"], A=32, state_dim=32, T=c["steps"], pos_base=P, pad_start=0, pad_end=0,
                    self_every=max(c["self_every"], 1), act_bf16=0, rms_eps=c["rms_eps"], rope_base=c["rope_base"],
                    min_period=c["min_period"], max_period=c["max_period"])
        self.model = orc.DenoiseModel(ocfg, ow)
        self.kp = [rng.standard_normal((P, c["n_kv"], hd), dtype=np.float32) for _ in range(L)]
        self.vp = [rng.standard_normal((P, c["n_kv"], hd), dtype=np.float32) for _ in range(L)]
        self.rng = rng

    def run(self, n_obs):
        """Seconds per observation for n_obs observations (inputs drawn before the clock starts)."""
        xs = [(self.rng.standard_normal(32).astype(np.float32), self.rng.standard_normal((50, 32)).astype(np.float32))
              for _ in range(n_obs)]
        times = []
        for state, x0 in xs:
            t0 = time.perf_counter()
            out = self.model.denoise(self.kp, self.vp, state, x0)
            times.append(time.perf_counter() - t0)
            assert np.isfinite(out).all()
        return times


PI0 = dict(model=0, n_layers=18, H=1024, n_q=8, n_kv=1, head_dim=256, inter=4096, chunk=50, action_dim=32,
           state_dim=32, steps=10, self_every=1, rms_eps=1e-6, rope_base=10000.0, min_period=4e-3, max_period=4.0)
PI0_P = 816
# SmolVLA-shaped action expert (BASELINE configs[0]): hidden 720, 16 layers alternating self- / cross-attention,
# 15 q / 5 kv heads of 64, MLP 2048, prefix 177, the state token lives in the prefix (suffix = 50 action tokens)
SMOLVLA = dict(model=1, n_layers=16, H=720, n_q=15, n_kv=5, head_dim=64, inter=2048, chunk=50, action_dim=32,
               state_dim=32, steps=10, self_every=2, rms_eps=1e-5, rope_base=10000.0, min_period=4e-3, max_period=4.0)
SMOLVLA_P = 177
# pi0.5-shaped expert (src/models/pi05.cpp): pi0's sizes, adaptive RMSNorm, no state token
PI05 = dict(PI0, model=2, state_dim=0, cond_dim=1024)
POLICIES = {"pi0": (PI0, PI0_P), "smolvla": (SMOLVLA, SMOLVLA_P), "pi05": (PI05, PI0_P)}


def policy_flops_per_chunk(c, P):
    """Dense FLOPs of a policy's denoise loop per observation: expert GEMMs + attention (algorithmic)."""
    S = c["chunk"] + (1 if c["model"] == 0 else 0)
    qf, kvf, H, I = c["n_q"] * c["head_dim"], c["n_kv"] * c["head_dim"], c["H"], c["inter"]
    total = 0
    for l in range(c["n_layers"]):
        cross = c["model"] == 1 and c["self_every"] > 1 and l % c["self_every"] != 0
        proj = 2 * S * H * qf if cross else 2 * S * H * (qf + 2 * kvf)  # cross layers: K / V projected once per observation
        keys = P if cross else P + S
        total += proj + 2 * S * qf * H + 3 * 2 * S * H * I + 4 * S * c["n_q"] * keys * c["head_dim"]
    per_step = total + 2 * 2 * c["chunk"] * H * H
    return per_step * c["steps"]


def pi0_flops_per_chunk():
    """Dense FLOPs of the pi0-shaped loop per observation: expert GEMMs + attention (algorithmic)."""
    c, S = PI0, 51
    qf, kvf, H, I = c["n_q"] * c["head_dim"], c["n_kv"] * c["head_dim"], c["H"], c["inter"]
    per_layer = 2 * S * H * (qf + 2 * kvf) + 2 * S * qf * H + 3 * 2 * S * H * I + 4 * S * c["n_q"] * (PI0_P + S) * c["head_dim"]
    per_step = c["n_layers"] * per_layer + 2 * 2 * c["chunk"] * H * H
    return per_step * c["steps"]


def build_pi0_engine(torch, vb, dev, n_obs, seed, policy="pi0"):
    c, PI0_P = POLICIES[policy]
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    H, I, qf, kvf, A, sd = c["H"], c["inter"], c["n_q"] * c["head_dim"], c["n_kv"] * c["head_dim"], 32, 32
    bw = lambda *s: (torch.randn(s, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    fv = lambda n: torch.zeros(n, device=dev)
    L = c["n_layers"]
    cross = [c["model"] == 1 and c["self_every"] > 1 and l % c["self_every"] != 0 for l in range(L)]
    w = dict(wq=[bw(qf, H) for _ in range(L)], wk=[bw(kvf, kvf if cross[l] else H) for l in range(L)],
             wv=[bw(kvf, kvf if cross[l] else H) for l in range(L)],
             wo=[bw(H, qf) for _ in range(L)], wgate=[bw(I, H) for _ in range(L)], wup=[bw(I, H) for _ in range(L)],
             wdown=[bw(H, I) for _ in range(L)], ln_in=[torch.ones(H, device=dev) for _ in range(L)],
             ln_post=[torch.ones(H, device=dev) for _ in range(L)], w_sp=bw(H, sd), b_sp=fv(H), w_ain=bw(H, A),
             b_ain=fv(H), w_at1=bw(H, 2 * H), b_at1=fv(H), w_at2=bw(H, H), b_at2=fv(H),
             out_norm=torch.ones(H, device=dev), w_aout=bw(A, H), b_aout=fv(A))
    if c["model"] == 2:
        fw = lambda *s: torch.randn(s, device=dev, generator=g) * 0.02
        gate_one = lambda: torch.cat([torch.zeros(2 * H, device=dev), torch.ones(H, device=dev)])  # scale 0, shift 0, gate 1
        w.update(ada_in_w=[fw(3 * H, H) for _ in range(L)], ada_in_b=[gate_one() for _ in range(L)],
                 ada_post_w=[fw(3 * H, H) for _ in range(L)], ada_post_b=[gate_one() for _ in range(L)],
                 ada_final_w=fw(3 * H, H), ada_final_b=gate_one(), w_tin=fw(H, H), b_tin=fv(H), w_tout=fw(H, H), b_tout=fv(H))
    eng = vb.PolicyEngine(c, w, max_obs=n_obs, prefix_len=PI0_P)
    del w
    blk = 64
    for l in range(L):  # the prefix KV is written once per observation
        for o in range(0, n_obs, blk):
            n = min(blk, n_obs - o)
            eng.set_prefix(l, torch.randn((n, PI0_P, c["n_kv"], c["head_dim"]), device=dev, generator=g),
                           torch.randn((n, PI0_P, c["n_kv"], c["head_dim"]), device=dev, generator=g), obs0=o)
    x0 = torch.randn((n_obs, 50, 32), device=dev, generator=g)
    state = torch.randn((n_obs, 32), device=dev, generator=g) if c["model"] != 2 else None
    torch.cuda.synchronize()
    return eng, x0, state


def measure_pi0(torch, vb, dev, n_obs, steps, warmup, seed, barrier=None, allow_graph=False, policy="pi0",
                on_begin=None):
    """Times `steps` whole denoise loops over n_obs observations: device-resident and through host buffers."""
    eng, x0, state = build_pi0_engine(torch, vb, dev, n_obs, seed, policy)
    sync = barrier or torch.cuda.synchronize
    for _ in range(warmup):
        eng.denoise(x0, state)
    sync()
    if on_begin:
        on_begin()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    ev[0].record()
    for i in range(steps):
        eng.denoise(x0, state)
        ev[i + 1].record()
    sync()
    step_ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(steps)]
    x0h, sth = x0.cpu().pin_memory(), (state.cpu().pin_memory() if state is not None else None)
    outh = torch.empty_like(x0h).pin_memory()
    eng.denoise_host(x0h, sth, outh)
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n_e2e = max(2, min(steps, 3))
    e0.record()
    for _ in range(n_e2e):
        eng.denoise_host(x0h, sth, outh)
    e1.record()
    sync()
    graph_ms = None
    if n_obs <= 8 and allow_graph and not (n_obs == 1 and os.environ.get("VLAB200_CHUNK_LOOP") != "0"):
        # small batches on the launch-per-operator path are latency-bound (~1,600 launches per chunk): the same loop replayed as one CUDA graph
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                eng.denoise(x0, state)
            torch.cuda.current_stream().wait_stream(side)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                out_g = eng.denoise(x0, state)
            g.replay()
            torch.cuda.synchronize()
            if torch.equal(out_g, eng.denoise(x0, state)):
                g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                g0.record()
                for _ in range(max(steps, 5)):
                    g.replay()
                g1.record()
                torch.cuda.synchronize()
                graph_ms = g0.elapsed_time(g1) / max(steps, 5)
        except RuntimeError:
            graph_ms = None
    if vb.device_status() != 0:
        raise SystemExit("device status word reports a kernel failure")
    return {"total_ms": ev[0].elapsed_time(ev[-1]), "p50_ms": statistics.median(step_ms),
            "e2e_ms": e0.elapsed_time(e1) / n_e2e, "h2d": x0h.numel() * 4 + (sth.numel() * 4 if sth is not None else 0),
            "d2h": outh.numel() * 4,
            "graph_ms": graph_ms}


def measure_ternary(torch, vb, dev, steps, warmup, only=None):
    """BitVLA-shaped ternary linear layers (BASELINE configs[3]): per-token int8 act-quant + 2-bit
    ladder-packed weights; M in {1, 300, 4800} x the four LM shapes.  Rotating operand sets larger
    than L2 between timed launches."""
    shapes = [("q/o", 2560, 2560, 1), ("k/v", 640, 2560, 1), ("gate_up", 13824, 2560, 2), ("down", 2560, 6912, 1)]
    g = torch.Generator(device=dev)
    g.manual_seed(3)
    rows = []
    for name, N, K, ws_num in shapes:
        for M in (1, 300, 4800):
            if only and only != f"{name}:{M}":
                continue
            n_sets = max(2, int(160e6 // (N * K // 4 + M * K + M * N * 2)) + 1)
            n_sets = min(n_sets, 24)
            a = torch.randint(-127, 128, (n_sets, M, K), dtype=torch.int8, device=dev, generator=g)
            wp = torch.randint(0, 256, (n_sets, N * K // 4), dtype=torch.uint8, device=dev, generator=g)
            sc = torch.rand((n_sets, M), device=dev, generator=g) * 100 + 40
            ws = torch.rand((ws_num,), device=dev, generator=g) * 0.05 + 0.01
            out = torch.empty((n_sets, M, N), dtype=torch.bfloat16, device=dev)
            for i in range(warmup):
                vb.ternary_linear(a[i % n_sets], wp[i % n_sets], sc[i % n_sets], ws, N, out=out[i % n_sets])
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = max(steps, 10) * 2
            e0.record()
            for i in range(reps):
                vb.ternary_linear(a[i % n_sets], wp[i % n_sets], sc[i % n_sets], ws, N, out=out[i % n_sets])
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / reps
            row = {"layer": name, "M": M, "N": N, "K": K, "us": ms * 1e3, "tops": 2.0 * M * N * K / ms / 1e9,
                   "packed_weight_gbs": N * K / 4 / ms / 1e6}
            if M <= 300:
                # few rows: the launches above are bound by the host's launch rate; the same launches replayed as one
                # CUDA graph give the device-side time
                try:
                    side = torch.cuda.Stream()
                    side.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(side):
                        vb.ternary_linear(a[0], wp[0], sc[0], ws, N, out=out[0])
                    torch.cuda.current_stream().wait_stream(side)
                    gr = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gr):
                        for i in range(reps):
                            vb.ternary_linear(a[i % n_sets], wp[i % n_sets], sc[i % n_sets], ws, N, out=out[i % n_sets])
                    gr.replay()
                    torch.cuda.synchronize()
                    e0.record()
                    for _ in range(5):
                        gr.replay()
                    e1.record()
                    torch.cuda.synchronize()
                    gms = e0.elapsed_time(e1) / (5 * reps)
                    row.update({"us_cuda_graph": gms * 1e3, "packed_weight_gbs_cuda_graph": N * K / 4 / gms / 1e6})
                    del gr
                except RuntimeError:
                    pass
            rows.append(row)
            del a, wp, sc, out
    if vb.device_status() != 0:
        raise SystemExit("device status word reports a kernel failure")
    reference_cuda = None if only else time_reference_ternary(torch, vb, dev, shapes)
    int8_live = None if only else measure_int8_peak(torch, dev)
    big = max((r for r in rows if r["M"] == 4800), key=lambda r: r["tops"], default=rows[0])
    gbs = lambda r: r.get("packed_weight_gbs_cuda_graph", r["packed_weight_gbs"])
    gemv = max((r for r in rows if r["M"] == 1), key=gbs, default=rows[0])
    hbm_peak, kind = measured_peaks()
    return {"metric": "ternary x int8 GEMM throughput (BitVLA LM shapes)", "value": big["tops"], "unit": "TOPS",
            "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": big["us"] / 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int8 x ternary (int32 accumulate)", "data": "synthetic",
            "config": {"workload": "ternary: BASELINE configs[3], 4 LM shapes x M in {1, 300, 4800}",
                       "l2": "operand sets rotated (> 126 MB) between launches"},
            "roofline": {"kernel": "ternary_gemm_pair_kernel", "bound": "tensor", "achieved": big["tops"],
                         "peak": INT8_PEAK_TOPS, "unit": "TOPS", "frac": big["tops"] / INT8_PEAK_TOPS,
                         "peak_kind": "of measured (cuBLASLt int8, burst)", "traffic": None, "shape": big},
            "roofline_gemv": {"kernel": "ternary_gemv_kernel", "bound": "hbm", "achieved": gbs(gemv),
                              "peak": hbm_peak, "unit": "GB/s", "frac": gbs(gemv) / hbm_peak,
                              "peak_kind": f"of {kind}", "shape": gemv},
            "shapes": rows, "int8_peak_live": int8_live, "reference_cuda": reference_cuda}


def _median_launch_ms(torch, fn, warm=5, reps=20):
    """Median of `reps` individually timed launches after `warm` warm-ups: the timing method of the reference's
    own kernel check (tests/bitvla_gemm_check.cu:146-185); same operands every launch, so L2 stays warm."""
    ms = []
    for it in range(warm + reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        if it >= warm:
            ms.append(e0.elapsed_time(e1))
    return statistics.median(ms)


def _graph_launch_ms(torch, fn, reps=20, replays=5):
    """Device time per launch: `reps` launches captured into one CUDA graph and replayed (no host launch cost)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        for _ in range(reps):
            fn()
    gr.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        gr.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (replays * reps)


def reference_lib(name):
    """A reference-derived checker library built by oracle/Makefile (absent when the reference tree was not
    there at build time): used here only as the timed GPU baseline, never on the product path."""
    import ctypes

    path = os.path.join(ROOT, "oracle", "_ref", name)
    return ctypes.CDLL(path) if os.path.exists(path) else None


def time_reference_ternary(torch, vb, dev, shapes):
    """The reference's own CUDA kernels (bitlinear_int8xint2_m: the "wide" wmma kernel; bitlinear_int8xint2: its
    M = 1 kernel) on the same shapes and the same box, both sides timed with the reference's method."""
    import ctypes as C

    ref = reference_lib("libbitnet_ref.so")
    if ref is None:
        return None
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    gemv_shapes = {(2560, 2560), (13824, 2560), (2560, 6912)}  # the M = 1 kernel is instantiated for these only
    rows = []
    for name, N, K, ws_num in shapes:
        for M in (1, 300, 4800):
            if M == 1 and (N, K) not in gemv_shapes:
                continue
            a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev, generator=g)
            wp = torch.randint(0, 256, (N * K // 4,), dtype=torch.uint8, device=dev, generator=g)
            sc = torch.rand((M,), device=dev, generator=g) * 100 + 40
            ws = torch.rand((ws_num,), device=dev, generator=g) * 0.05 + 0.01
            out_r = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
            out_m = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
            fn = ref.bitlinear_int8xint2 if M == 1 else ref.bitlinear_int8xint2_m
            ptrs = [C.c_void_p(t.data_ptr()) for t in (a, wp, out_r, sc, ws)]
            run_ref = lambda: fn(*ptrs, M, N, K, C.c_void_p(torch.cuda.current_stream().cuda_stream))
            run_own = lambda: vb.ternary_linear(a, wp, sc, ws, N, out=out_m)
            if M <= 300:  # a few microseconds of device time: launch cost would decide a per-launch timing
                t_ref, t_own, how = _graph_launch_ms(torch, run_ref), _graph_launch_ms(torch, run_own), "cuda graph replay"
            else:
                t_ref, t_own, how = _median_launch_ms(torch, run_ref), _median_launch_ms(torch, run_own), "median of 20 launches"
            same = bool((out_r.view(torch.int16).int() - out_m.view(torch.int16).int()).abs().max().item() <= 1)
            rows.append({"layer": name, "M": M, "N": N, "K": K, "reference_us": t_ref * 1e3, "this_library_us": t_own * 1e3,
                         "speedup": t_ref / t_own, "reference_tops": 2.0 * M * N * K / t_ref / 1e9, "timing": how,
                         "outputs_within_1_bf16_ulp": same})
    return {"kernel": "reference bitlinear_int8xint2_m (wide wmma kernel) / bitlinear_int8xint2 (M = 1), compiled "
                      "unmodified for sm_100", "method": "M = 4800: median of 20 launches after 5 warm-ups (the reference's own "
                      "method); M <= 300: 20 launches replayed as one CUDA graph; same operands each launch (L2 warm), both sides "
                      "timed the same way", "shapes": rows}


def measure_bitvla_lm(torch, vb, dev, steps, warmup, n_layers=30):
    """BitVLA-shaped language-model stack (hidden 2560, 20 q / 5 kv heads of 128, ffn 6912): every layer
    is norm+quant -> ternary q/k/v -> RoPE -> attention -> norm+quant -> ternary o -> norm+quant ->
    ternary gate_up -> gate*up+norm+quant -> ternary down.  Random packed weights (520 MB for 30 layers,
    larger than L2), 300-token sequences, 1 and 16 sequences per call."""
    hidden, n_q, n_kv, hd, ffn = 2560, 20, 5, 128, 6912
    hq, hkv = n_q * hd, n_kv * hd
    g = torch.Generator(device=dev)
    g.manual_seed(11)

    def pack(n, k):
        return torch.randint(0, 256, (n * k // 4,), dtype=torch.uint8, device=dev, generator=g)

    def scale(k, n=1):
        return (torch.rand((n,), device=dev, generator=g) * 0.4 + 0.8) / (2.0 * k / 3.0) ** 0.5

    def norm(k):
        return (torch.rand((k,), device=dev, generator=g) * 0.4 + 0.8).bfloat16()

    layers = []
    for _ in range(n_layers):
        layers.append({"attn_norm_w": norm(hidden), "attn_sub_norm_w": norm(hq), "ffn_norm_w": norm(hidden),
                       "ffn_sub_norm_w": norm(ffn), "q_packed": pack(hq, hidden), "q_ws": scale(hidden),
                       "k_packed": pack(hkv, hidden), "k_ws": scale(hidden), "v_packed": pack(hkv, hidden),
                       "v_ws": scale(hidden), "o_packed": pack(hidden, hq), "o_ws": scale(hq),
                       "gate_up_packed": pack(2 * ffn, hidden), "gate_up_ws": scale(hidden, 2),
                       "down_packed": pack(hidden, ffn), "down_ws": scale(ffn)})
    seq, max_batch = 300, 16
    lm = vb.BitvlaLM(hidden, n_q, n_kv, hd, ffn, layers, norm(hidden), rope_base=500000.0, rms_eps=1e-5, max_seq=seq,
                     max_batch=max_batch)
    macs_per_token = n_layers * (hidden * (hq + 2 * hkv) + hq * hidden + hidden * 2 * ffn + ffn * hidden)
    rows = []
    for n_seq in (1, max_batch):
        x = torch.randn((n_seq, seq, hidden), device=dev, generator=g).bfloat16()
        out = torch.empty_like(x)
        for _ in range(warmup):
            lm.forward(x, out)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            lm.forward(x, out)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        if not torch.isfinite(out.float()).all():
            raise SystemExit("non-finite output")
        rows.append({"n_seq": n_seq, "seq": seq, "ms": ms, "tokens_per_s": n_seq * seq / ms * 1e3,
                     "ternary_tops": 2.0 * macs_per_token * n_seq * seq / ms / 1e9,
                     "launches": 1 + 9 * n_layers + 1})
    # one token through the 30 layers: every ternary linear takes the packed-weight GEMV path, so the floor is the
    # 521 MB of packed weights crossing HBM once (launch- and latency-bound in practice: 9 small kernels per layer)
    x1 = torch.randn((1, 1, hidden), device=dev, generator=g).bfloat16()
    o1 = torch.empty_like(x1)
    for _ in range(warmup):
        lm.forward(x1, o1)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(max(steps, 10)):
        lm.forward(x1, o1)
    e1.record()
    torch.cuda.synchronize()
    ms1 = e0.elapsed_time(e1) / max(steps, 10)
    try:
        ms1_graph = _graph_launch_ms(torch, lambda: lm.forward(x1, o1), reps=1, replays=10)
    except RuntimeError:
        ms1_graph = None
    packed_bytes = n_layers * (hq * hidden + 2 * hkv * hidden + hidden * hq + 2 * ffn * hidden + hidden * ffn) / 4
    hbm_peak, hbm_kind = measured_peaks()
    one_token = {"ms": ms1, "packed_weight_bytes": packed_bytes, "packed_weight_gbs": packed_bytes / ms1 / 1e6,
                 "frac_of_hbm": packed_bytes / ms1 / 1e6 / hbm_peak, "peak_kind": f"of {hbm_kind}",
                 "ms_cuda_graph": ms1_graph,
                 "frac_of_hbm_cuda_graph": packed_bytes / ms1_graph / 1e6 / hbm_peak if ms1_graph else None,
                 "launches": 1 + 9 * n_layers + 1}
    if vb.device_status() != 0:
        raise SystemExit("device status word reports a kernel failure")
    reference_cuda = time_reference_lm(torch, dev, layers, norm(hidden), hidden, n_q, n_kv, hd, ffn, seq, rows[0]["ms"])
    big = rows[-1]
    return {"metric": "BitVLA LM stack throughput", "value": big["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1,
            "steps": steps, "warmup": warmup, "ms_per_step": big["ms"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 x ternary (int32 accumulate), bf16 between the linears",
            "data": "synthetic",
            "config": {"workload": f"bitvla_lm: {n_layers} BitNet layers, hidden 2560, 20q/5kv x 128, ffn 6912, "
                                   f"{max_batch} sequences x {seq} tokens per call",
                       "l2": "520 MB of packed weights streamed per call (> 126 MB L2)"},
            "gpu_launches": big["launches"] * steps,
            "roofline": {"kernel": "ternary_gemm_pair_kernel (whole stack, all kernels' time in the denominator)",
                         "bound": "tensor", "achieved": big["ternary_tops"], "peak": INT8_PEAK_TOPS, "unit": "TOPS",
                         "frac": big["ternary_tops"] / INT8_PEAK_TOPS,
                         "peak_kind": "of measured (cuBLASLt int8, burst)", "traffic": None},
            "cases": rows, "one_token": one_token, "reference_cuda": reference_cuda}


def time_reference_lm(torch, dev, layers, out_norm, hidden, n_q, n_kv, hd, ffn, seq, own_ms_one_seq):
    """The reference's bitvla_lm_cuda_forward (cuBLAS attention + its ternary kernels, one sequence per call) on
    the same weights, timed on the same box."""
    import ctypes as C

    ref = reference_lib("libbitvla_lm_ref.so")
    if ref is None:
        return None
    fields = ["attn_norm_w", "attn_sub_norm_w", "ffn_norm_w", "ffn_sub_norm_w", "q_packed", "q_ws", "k_packed", "k_ws",
              "v_packed", "v_ws", "o_packed", "o_ws", "gate_up_packed", "gate_up_ws", "down_packed", "down_ws"]

    class LayerC(C.Structure):
        _fields_ = [(n, C.c_void_p) for n in fields]

    ref.bitvla_lm_cuda_init.restype = C.c_void_p
    ref.bitvla_lm_cuda_init.argtypes = [C.c_int] * 6 + [C.c_float, C.c_float, C.c_int]
    ref.bitvla_lm_cuda_set_layer.argtypes = [C.c_void_p, C.c_int, C.POINTER(LayerC)]
    ref.bitvla_lm_cuda_set_output_norm.argtypes = [C.c_void_p, C.c_void_p]
    ref.bitvla_lm_cuda_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    ref.bitvla_lm_cuda_free.argtypes = [C.c_void_p]
    ctx = ref.bitvla_lm_cuda_init(hidden, n_q, n_kv, hd, ffn, len(layers), 500000.0, 1e-5, seq)
    if not ctx:
        return None
    for i, lw in enumerate(layers):
        st = LayerC(**{n: lw[n].data_ptr() for n in fields})
        ref.bitvla_lm_cuda_set_layer(ctx, i, C.byref(st))
    ref.bitvla_lm_cuda_set_output_norm(ctx, out_norm.data_ptr())
    x = torch.randn((seq, hidden), device=dev).bfloat16()
    out = torch.empty_like(x)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    run = lambda: ref.bitvla_lm_cuda_forward(ctx, x.data_ptr(), out.data_ptr(), seq, stream)
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 5
    ref.bitvla_lm_cuda_free(ctx)
    return {"kernel": "reference bitvla_lm_cuda_forward, compiled unmodified for sm_100 (one sequence per call)",
            "seq": seq, "ms": ms, "tokens_per_s": seq / ms * 1e3, "this_library_ms_one_sequence": own_ms_one_seq,
            "speedup_one_sequence": ms / own_ms_one_seq}


def measure_bitvla_vit(torch, vb, dev, n_layers=26):
    """The BitVLA vision tower (26 ternary ViT layers, hidden 1152, 16 heads of 72, MLP 4304, 256 patches, projector to
    2560) for one image through bitvla_vit_cuda_forward of this library and, where it was built, of the reference
    (oracle/_ref/libbitvla_vit_ref.so: its CUDA sources compiled unmodified), same weights, same box."""
    import ctypes as C

    H, heads, F, S, P, M = 1152, 16, 4304, 256, 588, 2560
    FP = (F + 127) // 128 * 128
    fields = ["ln1_w", "ln1_b", "ln2_w", "ln2_b", "q_packed", "q_ws", "q_b", "k_packed", "k_ws", "k_b", "v_packed", "v_ws",
              "v_b", "o_packed", "o_ws", "o_b", "fc1_packed", "fc1_ws", "fc1_b", "fc2_packed", "fc2_ws", "fc2_b"]

    class LayerC(C.Structure):
        _fields_ = [(n, C.c_void_p) for n in fields]

    g = torch.Generator(device=dev)
    g.manual_seed(11)
    bf = lambda *shape, sc=1.0: (torch.randn(shape, device=dev, generator=g) * sc).bfloat16()
    layers = []
    for _ in range(n_layers):
        lw = {"ln1_w": 1 + bf(H, sc=0.1), "ln1_b": bf(H, sc=0.05), "ln2_w": 1 + bf(H, sc=0.1), "ln2_b": bf(H, sc=0.05)}
        for name, n, k in (("q", H, H), ("k", H, H), ("v", H, H), ("o", H, H), ("fc1", F, H), ("fc2", H, FP)):
            # uniform ternary codes 1..3 (-1, 0, +1) in the ladder layout: any byte pattern is a valid pack
            codes = torch.randint(1, 4, (n * k // 4, 4), device=dev, generator=g, dtype=torch.int32)
            lw[name + "_packed"] = (codes[:, 0] | (codes[:, 1] << 2) | (codes[:, 2] << 4) | (codes[:, 3] << 6)).to(torch.uint8)
            lw[name + "_ws"] = torch.full((1,), (1.5 / k) ** 0.5, device=dev, dtype=torch.float32)
            lw[name + "_b"] = bf(n, sc=0.05)
        layers.append(lw)
    glob = dict(patch_w=bf(H, P, sc=P ** -0.5), patch_b=bf(H, sc=0.05), pos=bf(S, H, sc=0.1), w1=bf(M, H, sc=H ** -0.5),
                b1=bf(M, sc=0.05), w2=bf(M, M, sc=M ** -0.5), b2=bf(M, sc=0.05))
    patches = (torch.rand((S, P), device=dev, generator=g) * 2 - 1).bfloat16()
    out = torch.empty((S, M), device=dev, dtype=torch.bfloat16)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def timed(lib):
        lib.bitvla_vit_cuda_init.restype = C.c_void_p
        lib.bitvla_vit_cuda_init.argtypes = [C.c_int] * 6 + [C.c_float, C.c_int]
        lib.bitvla_vit_cuda_free.argtypes = [C.c_void_p]
        lib.bitvla_vit_cuda_set_layer.argtypes = [C.c_void_p, C.c_int, C.POINTER(LayerC)]
        lib.bitvla_vit_cuda_set_embed.argtypes = [C.c_void_p] * 4
        lib.bitvla_vit_cuda_set_mmproj.argtypes = [C.c_void_p] * 5
        lib.bitvla_vit_cuda_forward.restype = C.c_int
        lib.bitvla_vit_cuda_forward.argtypes = [C.c_void_p] * 4
        ctx = lib.bitvla_vit_cuda_init(n_layers, H, heads, F, S, P, 1e-6, M)
        if not ctx:
            return None
        for i, lw in enumerate(layers):
            st = LayerC(**{n: lw[n].data_ptr() for n in fields})
            lib.bitvla_vit_cuda_set_layer(ctx, i, C.byref(st))
        lib.bitvla_vit_cuda_set_embed(ctx, glob["patch_w"].data_ptr(), glob["patch_b"].data_ptr(), glob["pos"].data_ptr())
        lib.bitvla_vit_cuda_set_mmproj(ctx, glob["w1"].data_ptr(), glob["b1"].data_ptr(), glob["w2"].data_ptr(), glob["b2"].data_ptr())
        run = lambda: lib.bitvla_vit_cuda_forward(ctx, patches.data_ptr(), out.data_ptr(), stream)
        assert run() == 0
        torch.cuda.synchronize()
        ms = _median_launch_ms(torch, run, warm=3, reps=10)
        lib.bitvla_vit_cuda_free(ctx)
        return ms

    ours = timed(vb.lib())
    assert vb.device_status() == 0 and bool(torch.isfinite(out.float()).all())
    rec = {"config": f"BitVLA vision tower: {n_layers} ternary ViT layers, hidden {H}, {heads} heads of {H // heads}, MLP {F}, "
                     f"{S} patches, projector to {M}; one image per call", "ms": ours, "launches": 3 + 10 * n_layers + 3}
    ref = reference_lib("libbitvla_vit_ref.so")
    ref_ms = timed(ref) if ref is not None else None
    if ref_ms:
        rec["reference_cuda"] = {"kernel": "reference bitvla_vit_cuda_forward, compiled unmodified for sm_100", "ms": ref_ms,
                                 "speedup": ref_ms / ours}
    return rec


def measure_bitvla_head(vb):
    """BitVLA's float32 action head (chunk 8, 7 action dims, hidden 2560: fc1 streams 183 MB of float32 weights) and
    proprioception projector through bitvla_fp32head_* of this library and of the reference (cuBLAS SGEMM), host
    buffers in, host buffers out, wall clock (the calls copy and synchronise themselves)."""
    import ctypes as C

    P, H, M, A = 8, 2560, 8, 7
    D = A * H
    rng = np.random.default_rng(3)
    shapes = [(H, P), (H,), (H, H), (H,), (D,), (D,), (H, D), (H,), (H,), (H,), (H, H), (H,), (H,), (H,), (H, H), (H,), (H,), (H,),
              (A, H), (A,)]
    ws = [(rng.standard_normal(shp, dtype=np.float32) * (shp[-1] ** -0.5 if len(shp) == 2 else 0.1)) for shp in shapes]
    state = rng.standard_normal(P, dtype=np.float32)
    ah_in = rng.standard_normal((M, D), dtype=np.float32)
    fp = lambda a: a.ctypes.data_as(C.POINTER(C.c_float))

    def timed(lib):
        f = C.POINTER(C.c_float)
        lib.bitvla_fp32head_cuda_init.restype = C.c_void_p
        lib.bitvla_fp32head_cuda_init.argtypes = [C.c_int] * 4 + [C.c_float] + [f] * 20
        lib.bitvla_fp32head_proprio_forward.argtypes = [C.c_void_p, f, f, C.c_void_p]
        lib.bitvla_fp32head_action_forward.argtypes = [C.c_void_p, f, f, C.c_void_p]
        lib.bitvla_fp32head_cuda_free.argtypes = [C.c_void_p]
        ctx = lib.bitvla_fp32head_cuda_init(P, H, M, A, 1e-5, *[fp(w) for w in ws])
        if not ctx:
            return None
        pp, act = np.zeros(H, np.float32), np.zeros((M, A), np.float32)
        res = {}
        for name, call in (("action_ms", lambda: lib.bitvla_fp32head_action_forward(ctx, fp(ah_in), fp(act), None)),
                           ("proprio_ms", lambda: lib.bitvla_fp32head_proprio_forward(ctx, fp(state), fp(pp), None))):
            ts = []
            for it in range(25):
                t0 = time.perf_counter()
                assert call() == 0
                if it >= 5:
                    ts.append((time.perf_counter() - t0) * 1e3)
            res[name] = statistics.median(ts)
        lib.bitvla_fp32head_cuda_free(ctx)
        return res

    rec = {"config": f"BitVLA float32 head: chunk {M} x {A} actions, hidden {H} (fc1 {H} x {D}), proprio {P}; host in, host out"}
    rec.update(timed(vb.lib()))
    # the action forward streams every weight once: 4 B x (H D + 2 H H + A H) and the two LayerNorm vectors
    wbytes = 4.0 * (H * D + 2 * H * H + A * H + 2 * D + 8 * H)
    rec["action_weight_stream_gbs"] = wbytes / (rec["action_ms"] * 1e-3) / 1e9
    ref = reference_lib("libbitvla_fp32head_ref.so")
    if ref is not None:
        r = timed(ref)
        if r:
            rec["reference_cuda"] = dict(r, kernel="reference bitvla_fp32head_*, compiled unmodified for sm_100",
                                         speedup_action=r["action_ms"] / rec["action_ms"])
    return rec


def attn_config_dict(batch, n_gpus):
    return {"workload": "smolvla_attn: isolated denoise-attention op (BASELINE configs[1]), 16 layers x 10 steps, "
                        "P=177, S=51, 15q/5kv, hd 64, bf16",
            "batch_per_gpu": batch, "global_batch": batch * n_gpus, "parallelism": f"replica x{n_gpus}",
            "l2": "inputs larger than L2 (KV store + hidden states > 126 MB per GPU)"}


def policy_config_dict(workload, n_obs, n_global, world):
    text = {"pi0": "pi0_loop: whole pi0-shaped denoise loop (BASELINE configs[4], shapes of configs[2]): 18 expert layers, "
                   "hidden 1024, 8q/1kv, hd 256, MLP 4096, prefix 816, chunk 50x32 + state token, 10 Euler steps; "
                   "1024 observations split over the GPUs",
            "smolvla": "smolvla_loop: whole SmolVLA-shaped denoise loop (the action expert of BASELINE configs[0]): 16 "
                       "layers alternating self / cross attention, hidden 720, 15q/5kv, hd 64, MLP 2048, prefix 177, "
                       "chunk 50x32, 10 Euler steps",
            "pi05": "pi05_loop: whole pi0.5-shaped denoise loop: pi0's expert sizes with adaptive RMSNorm on the time step, "
                    "gated residuals, no state token, no mask among the 50 action tokens; prefix 816, 10 Euler steps"}[workload]
    return {"workload": text, "batch_per_gpu": n_obs, "global_batch": n_global, "parallelism": f"replica x{world}",
            "l2": "inputs larger than L2 (KV pages + expert weights + activations > 126 MB per GPU)"}


def run_reference(args, rank, world):
    """The reference arm: the CPU restatement of the SAME loop on the host cores (the reference's own CPU
    path runs through ggml, which is not part of its source tree), one observation per step."""
    if rank != 0:
        return
    from oracle import oracle_ffi as orc

    # as the reference's default_cpu_threads() (src/arch.h:43-54): min(cores, 16), whatever the launcher exported
    orc.set_num_threads(min(os.cpu_count() or 1, 16))
    threads = orc.num_threads()
    if args.workload == "smolvla_attn":
        rng = np.random.default_rng(1)
        for _ in range(max(args.warmup, 0)):
            oracle_chunk(orc, rng, 1)
        times = [oracle_chunk(orc, rng, 1) for _ in range(args.steps)]
        config = attn_config_dict(1, 1)
        sample = "1 observation (chunk) per step: 10 steps x 16 layers of QKV+RoPE+attention"
    elif args.workload.endswith("_predict"):
        from vla_cpp_b200 import synth_gguf

        arch = args.workload.split("_")[0]
        d = dict(synth_gguf.SMOLVLA_DIMS if arch == "smolvla" else synth_gguf.PI0_DIMS)
        n_views = 2 if arch == "smolvla" else 3
        times = [sum(oracle_predict_seconds(orc, d, arch, n_views)) for _ in range(max(args.steps, 1))]
        config = {"workload": f"{arch}_predict: one whole request (vision tower per view, backbone prefill, denoise loop), batch 1"}
        sample = "1 whole request per step with float32 weights and activations"
    elif args.workload == "pi05":
        workload = "pi05"
        times = oracle_pi05_seconds(orc, *POLICIES["pi05"], n=args.steps)
        config = policy_config_dict(workload, 1, 1, 1)
        sample = "1 observation (chunk) per step through the whole loop (all layers, 10 Euler steps), float32"
    else:
        workload = args.workload if args.workload in POLICIES else "pi0"
        loop = OraclePolicyLoop(orc, workload, seed=1)
        loop.run(max(min(args.warmup, 2), 0))
        times = loop.run(args.steps)
        config = policy_config_dict(workload, 1, 1, 1)
        sample = ("1 observation (chunk) per step through the whole loop (all layers, 10 Euler steps) with float32 "
                  "weights and activations")
    total = sum(times)
    value = args.steps / total
    line = {
        "impl": "reference", "metric": "action chunks/s (denoise loop)", "value": value, "unit": "chunks/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "p50_chunk_latency_ms": 1e3 * statistics.median(times), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
        "cpu_baseline": {"value": value, "unit": "chunks/s", "cores": threads, "kind": "port",
                         "sample": sample + "; the reference's own CPU path needs ggml (llama.cpp b10331), absent here"},
        "e2e": {"value": value, "unit": "chunks/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def time_stage(torch, eng, stage, n_obs, n_layers, rounds=2):
    """Average device time (ms) of one launch of `stage`, walking the layers (each layer has its own weights and
    K/V pages, so consecutive launches do not find their operands in L2)."""
    for l in range(n_layers):
        eng.run_stage(l, stage, n_obs)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(rounds):
        for l in range(n_layers):
            eng.run_stage(l, stage, n_obs)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (rounds * n_layers)


def policy_stage_records(torch, eng, c, P, n_obs, peaks):
    """Per-stage timings of one expert layer at this batch, with the algorithmic FLOPs / bytes of each."""
    S = c["chunk"] + (1 if c["model"] == 0 else 0)
    M, H, I, hd = n_obs * S, c["H"], c["inter"], c["head_dim"]
    qf, kvf = c["n_q"] * hd, c["n_kv"] * hd
    flops = {"qkv": 2.0 * M * H * (qf + 2 * kvf), "attention": 4.0 * M * c["n_q"] * (P + S) * hd,
             "o_proj": 2.0 * M * qf * H, "gate_up": 2.0 * M * H * 2 * I, "down": 2.0 * M * I * H}
    out = {}
    for stage in ("qkv", "attention", "o_proj", "gate_up", "down"):
        ms = time_stage(torch, eng, stage, n_obs, c["n_layers"])
        out[stage] = {"us_per_launch": ms * 1e3, "tflops": flops[stage] / (ms * 1e-3) / 1e12}
    # attention: prefix K/V + suffix K/V + Q + O per observation per layer-step (algorithmic bytes)
    att_bytes = n_obs * 2.0 * ((P + S) * kvf * 2 + S * qf * 2)
    a = out["attention"]
    a.update({"algorithmic_bytes_per_launch": att_bytes, "hbm_gbs": att_bytes / (a["us_per_launch"] * 1e-6) / 1e9,
              "hbm_frac": att_bytes / (a["us_per_launch"] * 1e-6) / 1e9 / peaks["hbm_gbs"],
              "tensor_frac": a["tflops"] / peaks["bf16_tflops_sustained"],
              "flop_per_byte": flops["attention"] / att_bytes})
    return out, flops


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "kind": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "kind": "fallback"}


def measure_policy(torch, vb, dist, dev, args, rank, world, barrier):
    """The whole denoise loop (pi0- or SmolVLA-shaped) over 1024 observations split across the ranks."""
    from vla_cpp_b200.shard import shard_range

    workload = args.workload
    c, P = POLICIES[workload]
    n_obs = args.pi0_obs or shard_range(1024, world, rank)[1]
    n_global = args.pi0_obs * world if args.pi0_obs else 1024
    warmup = max(args.warmup, 3)
    peaks = load_peaks()
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    sampler.start()
    eng, x0, state = build_pi0_engine(torch, vb, dev, n_obs, 99 + rank, workload)
    for _ in range(warmup):
        eng.denoise(x0, state)
    barrier()
    sampler.mark_begin()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    ev[0].record()
    for i in range(args.steps):
        eng.denoise(x0, state)
        ev[i + 1].record()
    barrier()
    clocks = sampler.stop()
    step_ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
    total_ms = ev[0].elapsed_time(ev[-1])
    # ---- end to end: state / noise in pinned host memory, actions read back, every step -----------------
    x0h, sth = x0.cpu().pin_memory(), (state.cpu().pin_memory() if state is not None else None)
    outh = torch.empty_like(x0h).pin_memory()
    eng.denoise_host(x0h, sth, outh)
    barrier()
    n_e2e = max(2, min(args.steps, 5))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n_e2e):
        eng.denoise_host(x0h, sth, outh)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / n_e2e
    if not torch.isfinite(outh).all():
        raise SystemExit("non-finite action chunk")
    # ---- the stages of one expert layer, each timed alone on the launching stream -----------------------
    stages, flops = policy_stage_records(torch, eng, c, P, n_obs, peaks)
    if vb.device_status() != 0:
        raise SystemExit("device status word reports a kernel failure")
    stats = torch.tensor([total_ms, statistics.median(step_ms), e2e_ms, stages["gate_up"]["us_per_launch"],
                          stages["attention"]["us_per_launch"]], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    total_ms, p50_ms, e2e_ms, gu_us, att_us = [float(v) for v in stats.tolist()]
    if rank != 0:
        return None
    S = c["chunk"] + (1 if c["model"] == 0 else 0)
    loop_tf = policy_flops_per_chunk(c, P) * n_obs * args.steps / (total_ms * 1e-3) / 1e12  # per GPU (rank 0's share)
    gu_tf = flops["gate_up"] / (gu_us * 1e-6) / 1e12
    few = n_obs * S <= 256
    line = {
        "metric": "action chunks/s (denoise loop)", "value": n_global * args.steps / (total_ms * 1e-3),
        "unit": "chunks/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": total_ms / args.steps, "p50_chunk_latency_ms": p50_ms, "higher_is_better": True,
        "scaling": "weak" if args.pi0_obs else "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": policy_config_dict(workload, n_obs, n_global, world), "clocks": clocks,
        # per Euler step: 2 embedding kernels + 2 GEMMs, 5 kernels per layer (6 on the few-row path), head + Euler
        # (one observation: two rotation tables + the persistent loop kernel)
        "gpu_launches": (3 if n_obs == 1 and os.environ.get("VLAB200_CHUNK_LOOP") != "0"
                         else c["steps"] * (4 + c["n_layers"] * (6 if few else 5) + 2) + 3) * args.steps,
        "roofline": {"kernel": "dense_gemm_pair_kernel (fused RMSNorm + gate/up + activation, the loop's largest "
                               "share: M x 2*inter x H per layer-step)",
                     "bound": "tensor", "achieved": gu_tf, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                     "frac": gu_tf / peaks["bf16_tflops_sustained"],
                     "peak_kind": f"of {peaks['kind']} (sustained: the kernel is timed back to back over the layers)",
                     "traffic": None, "us_per_launch": gu_us, "algorithmic_flops_per_launch": flops["gate_up"]},
        "loop": {"tflops": loop_tf, "frac_of_sustained_bf16": loop_tf / peaks["bf16_tflops_sustained"],
                 "flops_per_chunk": policy_flops_per_chunk(c, P)},
        "stages": stages,
        # bytes of the whole job: every rank copies its own shard in and out
        "e2e": {"value": n_global / (e2e_ms * 1e-3), "unit": "chunks/s",
                "h2d_bytes_per_step": n_global * (c["chunk"] * 32 + 32) * 4, "d2h_bytes_per_step": n_global * c["chunk"] * 32 * 4,
                "ms_per_step": e2e_ms},
    }
    if n_obs == 1 and os.environ.get("VLAB200_CHUNK_LOOP") != "0":
        # one observation runs as ONE persistent kernel: its roofline is the stream of the expert's weights, once per Euler step
        wbytes = expert_weight_bytes(c) * c["steps"]
        ms = total_ms / args.steps
        gbs = wbytes / (ms * 1e-3) / 1e9
        line["stages_note"] = "stage records are the launch-per-operator kernels (vlab200_engine_run_stage), not what this run timed"
        line["roofline"] = {"kernel": "chunk_loop_kernel (whole Euler loop of one observation, one cooperative launch per chunk)",
                            "bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                            "peak_kind": f"of {peaks['kind']}",
                            # ncu: 2,010 MB read + 15.7 MB written per launch for the SmolVLA-shaped expert (profiles/chunk_loop_smolvla_b1.md)
                            "traffic": 2026.1e6 if workload == "smolvla" else None,
                            "us_per_launch": ms * 1e3, "algorithmic_bytes_per_launch": wbytes}
    del eng, x0, state
    torch.cuda.empty_cache()
    return line


def expert_weight_bytes(c):
    """bf16 bytes of the expert's layer weights, streamed once per Euler step (cross-attention layers project q only)."""
    qf, kvf = c["n_q"] * c["head_dim"], c["n_kv"] * c["head_dim"]
    total = 0
    for l in range(c["n_layers"]):
        cross = c["model"] == 1 and c.get("self_every", 1) > 1 and l % c["self_every"] != 0
        total += c["H"] * (qf + (0 if cross else 2 * kvf)) + qf * c["H"] + 3 * c["H"] * c["inter"]
    return 2.0 * total


def small_batch_latency(torch, vb, dev, workload):
    """configs[2]: chunk latency at batch 1 and 64 (one GPU)."""
    c, P = POLICIES[workload]
    weight_bytes = expert_weight_bytes(c)
    out = {}
    for b in (1, 64):
        out[b] = measure_pi0(torch, vb, dev, b, 10 if b == 1 else 5, 3, 7 + b, policy=workload)
    # one observation again on the launch-per-operator path (the persistent loop kernel off), also replayed as a CUDA graph
    old_env = os.environ.get("VLAB200_CHUNK_LOOP")
    os.environ["VLAB200_CHUNK_LOOP"] = "0"
    try:
        ops = measure_pi0(torch, vb, dev, 1, 10, 3, 8, allow_graph=True, policy=workload)
    finally:
        if old_env is None:
            del os.environ["VLAB200_CHUNK_LOOP"]
        else:
            os.environ["VLAB200_CHUNK_LOOP"] = old_env
    peaks = load_peaks()
    return {"p50_chunk_latency_ms_batch1": out[1]["p50_ms"],
            "batch1_path": "persistent loop kernel (one cooperative launch per chunk)" if old_env != "0" else "launch per operator",
            "p50_chunk_latency_ms_batch1_operator_path": ops["p50_ms"],
            "p50_chunk_latency_ms_batch1_operator_path_cuda_graph": ops["graph_ms"],
            "batch1_weight_stream_frac": weight_bytes * c["steps"] / (out[1]["p50_ms"] * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "batch1_e2e_ms": out[1]["e2e_ms"],
            "p50_step_latency_ms_batch64": out[64]["p50_ms"], "chunks_per_s_batch64": 64 / (out[64]["p50_ms"] * 1e-3),
            "batch64_e2e_ms": out[64]["e2e_ms"]}


def measure_smolvla_attn(torch, vb, dist, dev, args, rank, world, barrier, with_e2e=True):
    """BASELINE configs[1]: the isolated denoise-attention op (16 layers x 10 steps of fused QKV+RoPE+append and
    attention over prefix + suffix K/V) at `args.batch` observations per GPU."""
    c, B = CFG, args.batch
    g = torch.Generator(device=dev)
    g.manual_seed(1234 + rank)
    store = vb.KvStore(c["L"], B, c["n_kv"], c["hd"], c["P"], c["S"], device=dev)
    for l in range(c["L"]):  # the prefix KV is written once per observation
        kp = torch.randn((B, c["P"], c["n_kv"], c["hd"]), device=dev, generator=g)
        vp = torch.randn((B, c["P"], c["n_kv"], c["hd"]), device=dev, generator=g)
        store.write_prefix(l, kp, vp)
    # the store write alone (float32 K, V in, bf16 pages out; every layer gets the last layer's values again)
    w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    w0.record()
    for l in range(c["L"]):
        store.write_prefix(l, kp, vp)
    w1.record()
    torch.cuda.synchronize()
    kvw_ms = w0.elapsed_time(w1) / c["L"]
    kvw_bytes = 2 * B * c["P"] * c["n_kv"] * c["hd"] * (4 + 2)
    n_rows = (c["n_q"] + 2 * c["n_kv"]) * c["hd"]
    wqkv = (torch.randn((c["L"], n_rows, c["H"]), device=dev, generator=g) * 0.02).to(torch.bfloat16)
    ln_w = torch.ones((c["L"], c["H"]), device=dev)
    x = torch.empty((c["T"], c["L"], B * c["S"], c["H"]), dtype=torch.bfloat16, device=dev)
    for t in range(c["T"]):
        x[t] = torch.randn((c["L"], B * c["S"], c["H"]), device=dev, generator=g).to(torch.bfloat16)
    op = vb.DenoiseAttn(store, c["H"], c["n_q"], c["S"], ln_w, wqkv, c["eps"], vb.MASK_CAUSAL)
    torch.cuda.synchronize()

    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        op.run(x)
    barrier()
    sampler.mark_begin()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    ev[0].record()
    for i in range(args.steps):
        op.run(x)
        ev[i + 1].record()
    barrier()
    clocks = sampler.stop()
    step_ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
    total_ms = ev[0].elapsed_time(ev[-1])
    if vb.device_status() != 0:
        raise SystemExit("device status word reports a kernel failure")

    # the two kernels alone, on the launching stream
    n_att = c["L"] * c["T"]
    for l in range(c["L"]):
        vb.attention(store, l, op.q, c["S"], c["n_q"], c["P"] + c["S"], vb.MASK_CAUSAL, out=op.out[l])
    torch.cuda.synchronize()
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a0.record()
    for i in range(n_att):
        l = i % c["L"]
        vb.attention(store, l, op.q, c["S"], c["n_q"], c["P"] + c["S"], vb.MASK_CAUSAL, out=op.out[l])
    a1.record()
    torch.cuda.synchronize()
    att_ms = a0.elapsed_time(a1) / n_att
    q0, q1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    q0.record()
    for i in range(n_att):
        l = i % c["L"]
        vb.qkv_rope_append(store, l, x[0, l], None, op.wqkv[l], op.rope, c["eps"], c["S"], c["n_q"], q_out=op.q)
    q1.record()
    torch.cuda.synchronize()
    qkv_ms = q0.elapsed_time(q1) / n_att

    e2e = None
    if with_e2e:
        x_host = torch.empty(x.shape, dtype=torch.bfloat16, pin_memory=True)
        x_host.copy_(x)
        out_host = torch.empty(op.out.shape, dtype=torch.bfloat16, pin_memory=True)
        for _ in range(2):
            op.run_host(x_host, out_host)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_e2e = max(3, min(args.steps, 5))
        e0.record()
        for _ in range(n_e2e):
            op.run_host(x_host, out_host)
        e1.record()
        barrier()
        e2e = {"ms": e0.elapsed_time(e1) / n_e2e, "h2d": x_host.numel() * 2, "d2h": out_host.numel() * 2}
        del x_host, out_host

    stats = torch.tensor([total_ms, statistics.median(step_ms), att_ms, qkv_ms, e2e["ms"] if e2e else 0.0],
                         device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    total_ms, p50_ms, att_ms, qkv_ms, e2e_ms = [float(v) for v in stats.tolist()]
    if rank != 0:
        return None
    hbm_peak, peak_kind = measured_peaks()
    att_gbs = ATTN_BYTES_PER_OBS_LAYER_STEP * B / (att_ms * 1e-3) / 1e9
    line = {
        "metric": "action chunks/s (denoise loop)", "value": B * world * args.steps / (total_ms * 1e-3),
        "unit": "chunks/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": total_ms / args.steps, "p50_chunk_latency_ms": p50_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": attn_config_dict(B, world), "clocks": clocks, "gpu_launches": 2 * n_att * args.steps,
        "roofline": {"kernel": "attn_hd64_kernel", "bound": "hbm", "achieved": att_gbs, "peak": hbm_peak,
                     "unit": "GB/s", "frac": att_gbs / hbm_peak, "peak_kind": f"of {peak_kind}",
                     "traffic": ATTN_DRAM_BYTES_PER_OBS_NCU * B, "us_per_launch": att_ms * 1e3,
                     "algorithmic_bytes_per_launch": ATTN_BYTES_PER_OBS_LAYER_STEP * B},
        "kernels": {"attn_us": att_ms * 1e3, "qkv_rope_append_us": qkv_ms * 1e3,
                    "qkv_tflops": 2.0 * B * c["S"] * n_rows * c["H"] / (qkv_ms * 1e-3) / 1e12,
                    "kv_store_write_us": kvw_ms * 1e3, "kv_store_write_gbs": kvw_bytes / (kvw_ms * 1e-3) / 1e9},
    }
    if e2e:
        line["e2e"] = {"value": B * world / (e2e_ms * 1e-3), "unit": "chunks/s", "h2d_bytes_per_step": e2e["h2d"],
                       "d2h_bytes_per_step": e2e["d2h"], "ms_per_step": e2e_ms}
    del store, x, op, wqkv
    torch.cuda.empty_cache()
    return line


def measure_pi05_loop(torch, vb, dev, args):
    """The pi0.5-shaped loop on one GPU: device-resident and host-buffer timings of the whole loop (no per-stage hook:
    its layer has seven stages of its own)."""
    c, P = POLICIES["pi05"]
    n_obs = args.pi0_obs if args.pi0_obs > 0 else 1024
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    r = measure_pi0(torch, vb, dev, n_obs, args.steps, max(args.warmup, 3), 99, policy="pi05", on_begin=sampler.mark_begin)
    clocks = sampler.stop()
    peaks = load_peaks()
    per_step_ms = r["total_ms"] / args.steps
    tf = policy_flops_per_chunk(c, P) * n_obs / (per_step_ms * 1e-3) / 1e12
    line = {"metric": "action chunks/s (denoise loop)", "value": n_obs / (per_step_ms * 1e-3), "unit": "chunks/s", "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": per_step_ms, "p50_chunk_latency_ms": r["p50_ms"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": policy_config_dict("pi05", n_obs, n_obs, 1), "clocks": clocks,
            # per Euler step: embedding, 7 kernels per layer (+1 where a GEMM is cut along M), norm + head + Euler
            "gpu_launches": (3 if n_obs == 1 and os.environ.get("VLAB200_CHUNK_LOOP") != "0"
                             else c["steps"] * (1 + c["n_layers"] * 7 + 3) + 3) * args.steps,
            "e2e": {"value": n_obs / (r["e2e_ms"] * 1e-3), "unit": "chunks/s", "h2d_bytes_per_step": r["h2d"],
                    "d2h_bytes_per_step": r["d2h"]},
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                         "frac": tf / peaks["bf16_tflops_sustained"], "traffic": None,
                         "note": "whole loop (expert GEMMs + attention, algorithmic FLOPs) over its device time", "peak_source": peaks["kind"]}}
    if n_obs > 1:
        line.update({k: v for k, v in small_batch_latency(torch, vb, dev, "pi05").items() if "batch1" in k})
    return line


def predict_inputs(d, arch):
    """The request of BASELINE configs[0] (SmolVLA: 2 views, 48 token ids) / configs[2] (pi0: 3 views, 48 token ids),
    seeds 0..3 for the images, the tokens, the state and the noise."""
    side = d["image_size"]
    n_views = 2 if arch == "smolvla" else 3
    images = [np.random.default_rng(v).integers(0, 256, (side, side, 3), dtype=np.uint8) for v in range(n_views)]
    lang = np.random.default_rng(1).integers(0, d["vocab_size"], d["tokenizer_max_length"]).astype(np.int32)
    state = np.random.default_rng(2).standard_normal(d["max_state_dim"]).astype(np.float32)
    noise = np.random.default_rng(3).standard_normal((d["chunk_size"], d["max_action_dim"])).astype(np.float32)
    return images, lang, state, noise


def oracle_pi05_seconds(orc, c, P, n=1):
    """Seconds per observation of the CPU restatement of the pi0.5-shaped loop (random weights of the expert's shapes)."""
    rng = np.random.default_rng(9)
    H, I, hd, L = c["H"], c["inter"], c["head_dim"], c["n_layers"]
    qf, kvf = c["n_q"] * hd, c["n_kv"] * hd
    w = lambda *shape: orc.bf16_round(rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02))
    z = lambda k: np.zeros(k, np.float32)
    gate_one = lambda: np.concatenate([z(2 * H), np.ones(H, np.float32)])
    layers = [dict(wq=w(qf, H), wk=w(kvf, H), wv=w(kvf, H), wo=w(H, qf), wgate=w(I, H), wup=w(I, H), wdown=w(H, I),
                   ada_in_w=w(3 * H, H), ada_in_b=gate_one(), ada_post_w=w(3 * H, H), ada_post_b=gate_one()) for _ in range(L)]
    ww = dict(layers=layers, w_ain=w(H, 32), b_ain=z(H), w_tin=w(H, H), b_tin=z(H), w_tout=w(H, H), b_tout=z(H),
              ada_final_w=w(3 * H, H), ada_final_b=gate_one(), w_aout=w(32, H), b_aout=z(32))
    cfg = dict(H=H, n_q=c["n_q"], n_kv=c["n_kv"], hd=hd, steps=c["steps"], rms_eps=c["rms_eps"], rope_base=c["rope_base"],
               min_period=c["min_period"], max_period=c["max_period"])
    kp = [rng.standard_normal((P, c["n_kv"], hd), dtype=np.float32) for _ in range(L)]
    vp = [rng.standard_normal((P, c["n_kv"], hd), dtype=np.float32) for _ in range(L)]
    times = []
    for _ in range(n):
        x0 = rng.standard_normal((c["chunk"], 32), dtype=np.float32)
        t0 = time.perf_counter()
        out = orc.pi05_denoise(kp, vp, x0, ww, cfg)
        times.append(time.perf_counter() - t0)
        assert np.isfinite(out).all()
    return times


def oracle_predict_seconds(orc, d, arch, n_views):
    """One whole request through the CPU restatement with random weights of the checkpoint's shapes: the vision tower per
    view, the backbone's prefill over the prefix, the denoise loop.  Returns (tower s, prefill s, denoise s)."""
    rng = np.random.default_rng(5)
    VH, VI, P = d["vit_hidden"], d["vit_inter"], d["patch_size"]
    g = d["image_size"] // P
    s = d["vit_pixel_shuffle"]
    w = lambda *shape: orc.bf16_round(rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02))
    one, z = (lambda n: np.ones(n, np.float32)), (lambda n: np.zeros(n, np.float32))
    tw = dict(patch_w=w(VH, 3, P, P), patch_b=z(VH), pos=w(g * g, VH), post_w=one(VH), post_b=z(VH),
              connector=w(d["hidden"], VH * s * s), connector_b=None,
              layers=[dict(ln1_w=one(VH), ln1_b=z(VH), ln2_w=one(VH), ln2_b=z(VH), wq=w(VH, VH), bq=z(VH), wk=w(VH, VH),
                           bk=z(VH), wv=w(VH, VH), bv=z(VH), wo=w(VH, VH), bo=z(VH), fc1=w(VI, VH), b1=z(VI), fc2=w(VH, VI),
                           b2=z(VH)) for _ in range(d["vit_layers"])])
    tcfg = dict(image=d["image_size"], patch=P, hidden=VH, n_heads=d["vit_heads"], shuffle=s, ln_eps=d["vit_ln_eps"], out_scale=0.0)
    img = rng.integers(0, 256, (d["image_size"], d["image_size"], 3), dtype=np.uint8)
    t0 = time.perf_counter()
    for _ in range(n_views):
        emb = orc.siglip_tower(img, tw, tcfg)
    t_tower = time.perf_counter() - t0
    H, I, hd = d["hidden"], d["intermediate"], d["head_dim"]
    qf, kvf = d["n_q_heads"] * hd, d["n_kv_heads"] * hd
    layers = [dict(ln_in=one(H), wqkv=w(qf + 2 * kvf, H), wo=w(H, qf), ln_post=one(H), wgate=w(I, H), wup=w(I, H), wdown=w(H, I))
              for _ in range(d["n_layers"])]
    n_prefix = n_views * emb.shape[0] + d["tokenizer_max_length"] + (1 if arch == "smolvla" else 0)
    x = rng.standard_normal((n_prefix, H), dtype=np.float32)
    ocfg = dict(n_q=d["n_q_heads"], n_kv=d["n_kv_heads"], hd=hd, rms_eps=1e-5, rope_base=10000.0,
                act="silu" if arch == "smolvla" else "gelu")
    t0 = time.perf_counter()
    orc.vlm_prefill(x, layers, ocfg)
    t_prefill = time.perf_counter() - t0
    if arch == "pi05":
        t_denoise = oracle_pi05_seconds(orc, POLICIES["pi05"][0], n_prefix)[0]
    else:
        t_denoise = OraclePolicyLoop(orc, arch, seed=7).run(1)[0]
    return t_tower, t_prefill, t_denoise


def predict_launches(d, arch):
    """Kernels of one request, counted from the host code: tower (patchify, stream init, patch GEMM; 8 per layer;
    post-LayerNorm, connector, pi0's scale), prefix embeddings, prefill (tables, 2 per layer for q|k|v + rotation, 4 more
    on every layer but the last, 4 for the K/V projection of a cross-attention layer), denoise loop (one persistent kernel;
    VLAB200_CHUNK_LOOP=0: the few-row path, a launch per operator)."""
    L = d["n_layers"]
    every = d.get("self_attn_every_n_layers", 0) if arch == "smolvla" else 0
    cross = sum(1 for i in range(L) if every > 1 and i % every != 0)
    tower = 3 + 8 * d["vit_layers"] + 2 + (0 if arch == "smolvla" else 1)
    embed = 3 if arch == "smolvla" else 2
    prefill = 2 + 2 * L + 4 * (L - 1) + 4 * cross
    denoise = d["num_steps"] * ((3 if arch == "smolvla" else 4) + L * 6 + 2) + 2  # pi0: + the state-token kernel; 2 RoPE tables
    if os.environ.get("VLAB200_CHUNK_LOOP") != "0":
        denoise = 3  # one observation: two rotation tables + the persistent loop kernel
    return tower + embed + prefill + denoise


def measure_predict(torch, vb, dev, args, arch):
    """Whole requests through include/vla.h on a random-init checkpoint of the named shape: camera views (host, uint8)
    -> vision tower -> backbone prefill -> denoise loop -> actions (host).  One step = one vla_predict call."""
    import shutil
    import tempfile

    from vla_cpp_b200 import synth_gguf

    tmp = tempfile.mkdtemp(prefix="vla_b200_bench_")
    try:
        path = os.path.join(tmp, arch + "_random.gguf")
        t0 = time.perf_counter()
        dims = {} if arch == "smolvla" else {"vocab_size": 32768}  # pi0 / pi0.5: a 32k-row embedding table bounds the file size
        d = synth_gguf.write_checkpoint(path, arch, dims=dims, seed=0, matrix_dtype="f32" if arch == "smolvla" else "bf16")
        t_write = time.perf_counter() - t0
        t0 = time.perf_counter()
        model = vb.VlaModel(path)
        images, lang, state, noise = predict_inputs(d, arch)
        first = model.predict(lang, state, images=images, noise=noise)  # creates the device side on first use
        t_load = time.perf_counter() - t0
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    assert np.isfinite(first).all() and first.shape == (d["chunk_size"], d["max_action_dim"])
    for _ in range(max(args.warmup, 3)):
        model.predict(lang, state, images=images, noise=noise)
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    sampler.mark_begin()
    wall, phases = [], []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        out = model.predict(lang, state, images=images, noise=noise)
        wall.append((time.perf_counter() - t0) * 1e3)
        st = model.stats
        phases.append((st.ms_vision, st.ms_prefill, st.ms_denoise))
    clocks = sampler.stop()
    assert np.array_equal(out, first)  # same request, same noise: bit-identical actions
    med = lambda xs: float(statistics.median(xs))
    ms_v, ms_p, ms_d = (med([ph[i] for ph in phases]) for i in range(3))
    dev_ms, wall_ms = ms_v + ms_p + ms_d, med(wall)
    peaks = load_peaks()
    # weights streamed per request: tower and backbone once, expert once per Euler step (bf16 on the device)
    VH, VI = d["vit_hidden"], d["vit_inter"]
    tower_p = d["vit_layers"] * (4 * VH * VH + 2 * VH * VI) + d["hidden"] * VH * d["vit_pixel_shuffle"] ** 2
    hd = d["head_dim"]
    qf, kvf, H, I, E, EI = d["n_q_heads"] * hd, d["n_kv_heads"] * hd, d["hidden"], d["intermediate"], d["expert_h"], d["expert_inter"]
    backbone_p = d["n_layers"] * (H * (2 * qf + 2 * kvf) + 3 * H * I)
    expert_p = d["n_layers"] * (E * (2 * qf + 2 * kvf) + 3 * E * EI)
    bytes_alg = 2.0 * (tower_p + backbone_p + d["num_steps"] * expert_p)
    h2d = sum(a.nbytes for a in images) + lang.nbytes + state.nbytes + noise.nbytes
    line = {
        "metric": "action chunks/s and p50 chunk latency (whole request: vision tower + prefill + denoise loop)",
        "value": 1e3 / dev_ms, "unit": "chunks/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": dev_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (random-init checkpoint in the reference's GGUF naming, seeded request)",
        "config": {"workload": f"{arch}_predict: {'BASELINE configs[0]' if arch == 'smolvla' else 'shapes of BASELINE configs[2]'} through vla_predict, batch 1, "
                               f"{len(images)} uint8 views of {d['image_size']}x{d['image_size']}, {lang.size} token ids, "
                               f"{d['num_steps']} Euler steps", "l2": "weights (> L2) re-read every request"},
        "phases_ms": {"vision": ms_v, "prefill": ms_p, "denoise": ms_d, "wall_p50": wall_ms, "wall_min": min(wall),
                      "host_overhead": wall_ms - dev_ms},
        "e2e": {"value": 1e3 / wall_ms, "unit": "chunks/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": int(out.nbytes),
                "ms_per_step": wall_ms},
        "roofline": {"bound": "hbm", "achieved": bytes_alg / (dev_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": bytes_alg / (dev_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "traffic": None,
                     "note": "weights streamed per request (tower + backbone once, expert per step) over the device time of "
                             "the whole request; a batch-1 request is launch- and latency-bound, not bandwidth-bound",
                     "peak_source": peaks["kind"]},
        "gpu_launches": predict_launches(d, arch) * args.steps, "clocks": clocks,
        "setup_s": {"write_checkpoint": t_write, "load_and_first_predict": t_load},
    }
    return line, d


def cpu_baseline_record(args, workload):
    """The CPU restatement of the benchmarked loop on this box's host cores: a bounded sample."""
    from oracle import oracle_ffi as orc

    orc.set_num_threads(min(os.cpu_count() or 1, 16))
    if workload == "smolvla_attn":
        rng = np.random.default_rng(7)
        t1 = oracle_chunk(orc, rng, 1)
        n = max(1, min(16, int(args.cpu_seconds / max(t1, 1e-3))))
        tn = oracle_chunk(orc, rng, n)
        return {"value": n / tn, "unit": "chunks/s", "cores": orc.num_threads(), "kind": "port",
                "sample": f"{n} observation(s) of the same workload (10 steps x 16 layers each)"}
    loop = OraclePolicyLoop(orc, workload, seed=7)
    t1 = loop.run(1)[0]
    n = max(1, min(8, int(args.cpu_seconds / max(t1, 1e-3))))
    times = loop.run(n)
    return {"value": n / sum(times), "unit": "chunks/s", "cores": orc.num_threads(), "kind": "port",
            "sample": f"{n} observation(s) through the whole loop (all layers x 10 Euler steps, float32), after one "
                      f"warm-up observation"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=256, help="observations per GPU (smolvla_attn workload)")
    ap.add_argument("--workload", default="pi0", choices=["pi0", "smolvla", "pi05", "smolvla_attn", "ternary", "bitvla_lm", "smolvla_predict", "pi0_predict",
                             "pi05_predict"],
                    help="pi0 (default): the whole pi0-shaped denoise loop, 1024 observations split over the GPUs "
                         "(BASELINE configs[4]); smolvla: the SmolVLA-shaped loop; smolvla_attn: the isolated "
                         "denoise-attention op (configs[1]); ternary / bitvla_lm: configs[3]")
    ap.add_argument("--gemm-tiling", type=int, default=0,
                    help="bf16 GEMM tiling inside the engine: 0 automatic, 1 128x256, 2 128x128, 3 CTA pairs, 4 128x64")
    ap.add_argument("--ternary-only", default=None,
                    help="ternary workload: run one case only, e.g. gate_up:4800 (for profiler captures)")
    ap.add_argument("--pi0-obs", type=int, default=0, help="observations per GPU for the loop workloads (0: 1024 / N)")
    ap.add_argument("--no-extras", action="store_true",
                    help="default run: skip the small-batch latencies and the configs[1] / configs[3] sub-records")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    ap.add_argument("--int8-peak", action="store_true", help="measure the int8 tensor-core peak (cuBLASLt) and exit")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    import vla_cpp_b200 as vb

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    vb.lib()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if args.int8_peak:
        if rank == 0:
            print(json.dumps(measure_int8_peak(torch, dev)), flush=True)
        return
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"  # keep stdout to the one JSON line
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def finish(line):
        if rank == 0 and line is not None:
            print(json.dumps(line), flush=True)
        if world > 1:
            dist.destroy_process_group()

    vb.set_gemm_tiling(args.gemm_tiling)
    if args.workload == "ternary":
        finish(measure_ternary(torch, vb, dev, args.steps, max(args.warmup, 3), args.ternary_only) if rank == 0 else None)
        return
    if args.workload == "bitvla_lm":
        line = None
        if rank == 0:
            line = measure_bitvla_lm(torch, vb, dev, args.steps, max(args.warmup, 3))
            line["vision_tower"] = measure_bitvla_vit(torch, vb, dev)
            line["fp32_head"] = measure_bitvla_head(vb)
        finish(line)
        return
    if args.workload == "pi05":
        line = None
        if rank == 0:
            line = measure_pi05_loop(torch, vb, dev, args)
            if not args.no_cpu_baseline:
                from oracle import oracle_ffi as orc

                ts = oracle_pi05_seconds(orc, *POLICIES["pi05"], n=2)
                line["cpu_baseline"] = {"value": len(ts) / sum(ts), "unit": "chunks/s", "cores": orc.num_threads(), "kind": "port",
                                        "sample": "2 observations of the same loop"}
        finish(line)
        return
    if args.workload.endswith("_predict"):
        line = None
        if rank == 0:
            arch = args.workload.split("_")[0]
            line, d = measure_predict(torch, vb, dev, args, arch)
            if not args.no_cpu_baseline:
                from oracle import oracle_ffi as orc

                tt, tp, td = oracle_predict_seconds(orc, d, arch, 2 if arch == "smolvla" else 3)
                line["cpu_baseline"] = {"value": 1.0 / (tt + tp + td), "unit": "chunks/s", "cores": orc.num_threads(), "kind": "port",
                                        "sample": "one whole request of the same shapes (random weights)",
                                        "seconds": {"vision": tt, "prefill": tp, "denoise": td}}
        finish(line)
        return
    if args.workload == "smolvla_attn":
        line = measure_smolvla_attn(torch, vb, dist, dev, args, rank, world, barrier, with_e2e=not args.no_e2e)
        if line is not None and world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_record(args, "smolvla_attn")
        finish(line)
        return

    line = measure_policy(torch, vb, dist, dev, args, rank, world, barrier)
    if line is not None and world == 1:
        if not args.no_extras:
            line.update(small_batch_latency(torch, vb, dev, args.workload))
            sub = argparse.Namespace(**vars(args))
            sub.steps, sub.warmup = 5, 3
            a = measure_smolvla_attn(torch, vb, dist, dev, sub, 0, 1, torch.cuda.synchronize, with_e2e=False)
            line["smolvla_attn"] = {"config": a["config"], "chunks_per_s": a["value"], "ms_per_step": a["ms_per_step"],
                                    "roofline": a["roofline"], "kernels": a["kernels"]}
            t = measure_ternary(torch, vb, dev, 5, 3)
            line["ternary"] = {k: t[k] for k in ("config", "roofline", "roofline_gemv", "shapes", "int8_peak_live",
                                                 "reference_cuda") if k in t}
            lm = measure_bitvla_lm(torch, vb, dev, 5, 3)
            line["bitvla_lm"] = {k: lm[k] for k in ("config", "roofline", "cases", "one_token", "reference_cuda") if k in lm}
            line["bitvla_lm"]["vision_tower"] = measure_bitvla_vit(torch, vb, dev)
            line["bitvla_lm"]["fp32_head"] = measure_bitvla_head(vb)
        if not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_record(args, args.workload)
    finish(line)


if __name__ == "__main__":
    main()
