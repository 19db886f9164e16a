#!/usr/bin/env python3
"""bench.py -- decode tok/s of the Qwen2.5-0.5B-architecture Q8_0 model, batch 1, on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one decoded token = one pass of the whole Q8_0 decode path (24 layers + final
norm + LM head + argmax) over one token of synthetic input.  Weights are random-init and
quantised to Q8_0 (llamatov_b200.synth); the prompt is 32 uniform random token ids.

Printed JSON line (rank 0):
  value        tok/s with everything resident in HBM: K replays of the captured step with the
               token loop on the device (embedding gather and argmax inside the graph), CUDA
               events on the replay stream, max over ranks; the MEDIAN of --repeats timed regions
               of K steps each (the reference's own protocol is the median of 6 runs of 100
               replays, bpd/kernelgen/referee/rms_quant_prod_ab.py:22-47), min and max beside it.
  e2e          tok/s through the reference-facing call GraphRunner.replay_token(tok): per
               token the host copies the step's input to the device from page-locked memory
               (the token id, 4 bytes, when the embedding table is a Q8_0 table and the step
               gathers the row itself; else the fp32 row, E*4 bytes), launches the graph,
               synchronises and reads the chosen token back (4 bytes).  Median of the repeats.
  tp           the tensor-parallel path (BASELINE config 4): Llama-3-8B-architecture decode, 4096
               positions of context, TP = number of ranks, batch 1 and batch 32 (one object per
               batch: tok/s, ms per step, fraction of ranks x HBM peak, all-reduce share, token
               match and largest logit gap against the same tokens at TP = 1).
  roofline     the decode step as a whole: algorithmic bytes of one token (34 bytes per 32 weights of
               every matrix + the fp32 KV rows read once per KV head) divided by the device time per
               token (CUDA events on the replay stream), against the measured HBM copy bandwidth;
               traffic = DRAM bytes of one token's launches from an ncu capture of this command.  The
               one launch that is bandwidth-bound by itself, the LM-head GEMV, is also timed alone.
  cpu_baseline the CPU port of the same path (oracle/) timed on this box's host cores on a
               bounded sample (N=1 only).
With N > 1 every rank runs an independent replica of the model (the 0.5B model does not
shard: 2 KV heads, 0.5 GB of weights); value is the sum of tokens over ranks / max time.

--impl reference times the CPU implementation on the host cores (rank 0 only).
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

ARCH = "qwen2.5-0.5b"
PROMPT_LEN = 32
METRIC = "decode tok/s (0.5B Q8_0, bs1)"
UNIT = "tok/s"

# dram__bytes_read.sum + dram__bytes_write.sum of ONE token's launches, from an ncu capture of
# this very command, keyed by step mode; None where not captured.
NCU_TRAFFIC = {"pdl": 530232064, "persistent": 526459648}


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        j = json.load(open(p))
        return float(j["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s)"


def gemv_shapes(cfg):
    """(M, K, launches per token) of every Q8_0 GEMV in one decode step."""
    E, F, V = cfg["n_embd"], cfg["n_ffn"], cfg["vocab"]
    nq = cfg["n_head"] * cfg["hd"]; nk = cfg["n_head_kv"] * cfg["hd"]
    L = cfg["n_layers"]
    return [(nq + 2 * nk, E, L), (E, nq, L), (2 * F, E, L), (E, F, L), (V, E, 1)]


def gemv_bytes(M, K, T=1):
    """Algorithmic bytes of one GEMV launch: 34 B per 32 weights + T*(4K + 4M)."""
    return M * (K // 32) * 34 + T * (4 * K + 4 * M)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,clocks.mem,clocks.max.mem")

    def __init__(self, index):
        self.index = index; self.lines = []; self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True); self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, mem, memx, reasons = [], [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
            try:
                mem.append(float(f[9])); memx.append(float(f[10]))
            except (ValueError, IndexError):
                pass
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm),
                "mem_mhz": float(np.median(mem)) if mem else None, "mem_max_mhz": max(memx) if memx else None}


def cpu_decode_baseline(model, prompt, budget_s=15.0, max_tokens=16):
    """tok/s of the CPU port (oracle engine, OpenMP over output rows) on a bounded sample."""
    from oracle import oracle as o
    from llamatov_b200 import synth
    try:
        o.set_threads(len(os.sched_getaffinity(0)))
    except AttributeError:
        o.set_threads(os.cpu_count() or 1)
    eng = o.OracleEngine(synth.oracle_model(model), max_seq=256)
    t0 = time.perf_counter()
    for tk in prompt:               # the same 32-token prompt as the GPU arm, token by token
        _, nxt = eng.step(tk)
    first = (time.perf_counter() - t0) / len(prompt)
    n = int(max(2, min(max_tokens, budget_s / max(first, 1e-3))))
    t0 = time.perf_counter()
    for i in range(n):
        _, nxt = eng.step(nxt)
    dt = time.perf_counter() - t0
    return {"value": n / dt, "unit": UNIT, "cores": o.num_threads(), "kind": "port",
            "sample": f"{n} greedy decode steps of the full {ARCH} model after the {len(prompt)}-token prompt "
                      f"(oracle/lt_oracle.c, OpenMP over output rows)"}


def run_reference(args, rank):
    """--impl reference: the CPU implementation of the path on the host cores."""
    if rank != 0:
        return
    from llamatov_b200 import synth
    model = synth.make_model(ARCH, seed=0)
    prompt = np.random.default_rng(0).integers(0, model["cfg"]["vocab"], size=PROMPT_LEN).tolist()
    from oracle import oracle as o
    try:
        o.set_threads(len(os.sched_getaffinity(0)))     # all host cores, whatever the launcher exported
    except AttributeError:
        o.set_threads(os.cpu_count() or 1)
    eng = o.OracleEngine(synth.oracle_model(model), max_seq=max(256, PROMPT_LEN + args.warmup + args.steps + 8))
    for tk in prompt:               # the same 32-token prompt as the GPU arm, token by token (untimed)
        _, nxt = eng.step(tk)
    for _ in range(args.warmup):
        _, nxt = eng.step(nxt)
    t0 = time.perf_counter()
    n = 0
    for _ in range(args.steps):
        _, nxt = eng.step(nxt); n += 1
        if time.perf_counter() - t0 > 120:
            break
    dt = time.perf_counter() - t0
    val = n / dt
    cb = {"value": val, "unit": UNIT, "cores": o.num_threads(), "kind": "port",
          "sample": f"{n} greedy decode steps of the full {ARCH} model on the host "
                    "(oracle/lt_oracle.c: the reference's arithmetic restated in C, OpenMP over rows; the "
                    "reference's own CPU path for this architecture is a torch script that needs its checkout)"}
    print(json.dumps({"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
                      "steps": n, "warmup": args.warmup, "ms_per_step": 1000.0 * dt / n, "higher_is_better": True,
                      "scaling": "weak", "vs_baseline": None, "dtype": "int8*int8->int32, fp32 accumulate",
                      "data": "synthetic",
                      "config": {"workload": f"{ARCH} Q8_0 decode, batch 1, {PROMPT_LEN}-token prompt, {n} greedy steps",
                                 "parallelism": "host cores"},
                      "cpu_baseline": cb,
                      "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def run_config0(args):
    """BASELINE config 0: the single Q8_0 GEMV y = W x, W 4864 x 896 (28 blocks per row, d = fp16(|N(0,1)| * 0.02),
    q ~ U{-127..127}), x ~ N(0,1) fp32[896], numpy default_rng(0).  Prints one JSON line: the GPU result against
    the CPU oracle (bit-exact target), against a float64 dequantise-and-dot, and against the reference's own
    compiled CPU path (bpd_qmatmul_q8_0_llamafile_cpu from oracle/_ref/libbpd_cpu.so, a different fp32 order and
    quantiser) where that library was built; the GEMV's steady-state bandwidth; the CPU path's time."""
    import torch
    from llamatov_b200 import _lib, synth
    from oracle import oracle as o
    M, K = 4864, 896
    nb = K // 32
    Wq, Wd, x = synth.gemv_case(M, K, seed=0)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    dWq = torch.from_numpy(Wq).cuda(); dWd = torch.from_numpy(Wd.view(np.int16)).cuda()
    dx = torch.from_numpy(x[0]).cuda()
    xq = torch.empty(K, dtype=torch.int8, device="cuda"); xd = torch.empty(nb, dtype=torch.int16, device="cuda")
    y = torch.empty(M, dtype=torch.float32, device="cuda")
    _lib.call("lt_quant_q8", dx.data_ptr(), xq.data_ptr(), xd.data_ptr(), K, 1, st)
    _lib.call("lt_q8_gemv", dWq.data_ptr(), dWd.data_ptr(), xq.data_ptr(), xd.data_ptr(), None, y.data_ptr(), M, K, 1, st)
    torch.cuda.synchronize()
    yg = y.cpu().numpy()
    oq, od = o.quant_q8(x[0])
    want = np.asarray(o.q8_gemv(Wq, Wd, oq, od, M, K), np.float32)
    quant_equal = bool(np.array_equal(xq.cpu().numpy(), oq) and np.array_equal(xd.cpu().numpy().view(np.uint16), od.view(np.uint16)))
    ulp = int(np.max(np.abs(yg.view(np.int32).astype(np.int64) - want.view(np.int32).astype(np.int64))))
    Wf = Wq.reshape(M, nb, 32).astype(np.float64) * Wd.reshape(M, nb, 1).astype(np.float64)
    y64 = Wf.reshape(M, K) @ x[0].astype(np.float64)
    den = float(np.max(np.abs(y64)))
    rel64 = float(np.max(np.abs(yg - y64)) / den)
    # steady-state bandwidth: captured chain over rotating copies (no launch finds its matrix in L2)
    R = 64
    Wqs = dWq.repeat(R, 1); Wds = dWd.repeat(R, 1)
    side = torch.cuda.Stream()

    def run(i):
        _lib.call("lt_q8_gemv", Wqs[i % R].data_ptr(), Wds[i % R].data_ptr(), xq.data_ptr(), xd.data_ptr(), None,
                  y.data_ptr(), M, K, 1, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    for i in range(3):
        run(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        for i in range(2 * R):
            run(i)
    with torch.cuda.stream(side):
        for _ in range(max(3, args.warmup)):
            g.replay()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            g.replay()
        e1.record()
    torch.cuda.synchronize()
    us = 1000.0 * e0.elapsed_time(e1) / (10 * 2 * R)
    peak, peak_src = _peaks()
    gbs = gemv_bytes(M, K) / (us * 1e-6) / 1e9
    out = {"metric": "Q8_0 GEMV HBM GB/s (4864x896, batch 1)", "value": gbs, "unit": "GB/s", "n_gpus": 1,
           "us_per_launch": us, "higher_is_better": True, "dtype": "int8*int8->int32, fp32 accumulate", "data": "synthetic",
           "config": {"workload": "single Q8_0 GEMV 4864x896, x ~ N(0,1), numpy default_rng(0)"},
           "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                        "traffic": None, "peak_source": peak_src},
           "parity": {"activation_quant_bytes_equal_oracle": quant_equal, "max_ulp_vs_oracle": ulp,
                      "max_rel_vs_float64_dequant_dot": rel64}}
    ref_so = os.path.join(ROOT, "oracle", "_ref", "libbpd_cpu.so")
    if os.path.exists(ref_so):
        L = ctypes.CDLL(ref_so)
        fn = L.bpd_qmatmul_q8_0_llamafile_cpu
        fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        fn.restype = None
        blocks = np.empty((M * nb, 34), np.uint8)
        blocks[:, :2] = Wd.view(np.uint8).reshape(M * nb, 2); blocks[:, 2:] = Wq.view(np.uint8).reshape(M * nb, 32)
        xa = np.ascontiguousarray(x[0], np.float32); ya = np.zeros(M, np.float32)
        fn(blocks.ctypes.data, xa.ctypes.data, ya.ctypes.data, M, 1, K)
        t0 = time.perf_counter(); n = 0
        while time.perf_counter() - t0 < 2.0:
            fn(blocks.ctypes.data, xa.ctypes.data, ya.ctypes.data, M, 1, K); n += 1
        dt = (time.perf_counter() - t0) / n
        out["parity"]["max_rel_vs_reference_cpu_path"] = float(np.max(np.abs(yg - ya)) / den)
        # the same GEMV in the CPU library's own quantiser and fold order (parity mode): bit-exact target
        xq2 = torch.empty(K, dtype=torch.int8, device="cuda"); xd2 = torch.empty(nb, dtype=torch.int16, device="cuda")
        y2 = torch.empty(M, dtype=torch.float32, device="cuda")
        _lib.call("lt_quant_q8_ggml", dx.data_ptr(), xq2.data_ptr(), xd2.data_ptr(), K, 1, st)
        _lib.call("lt_q8_gemm_ggml", dWq.data_ptr(), dWd.data_ptr(), xq2.data_ptr(), xd2.data_ptr(), y2.data_ptr(), M, K, 1, st)
        torch.cuda.synchronize()
        y2h = y2.cpu().numpy()
        out["parity"]["ggml_order_mode_max_ulp_vs_reference_cpu_path"] = int(np.max(np.abs(
            y2h.view(np.int32).astype(np.int64) - ya.view(np.int32).astype(np.int64))))
        out["cpu_baseline"] = {"value": gemv_bytes(M, K) / dt / 1e9, "unit": "GB/s", "cores": 1, "kind": "reference",
                               "sample": f"{n} calls of bpd_qmatmul_q8_0_llamafile_cpu (bpd-substrate/bench/bpd_cpu.c:4419, "
                                         "single-threaded) on the same matrix", "us_per_call": dt * 1e6}
    print(json.dumps(out))


def run_tp_leg(rank, world, steps):
    """BASELINE config 4 on the ranks of this run: Llama-3-8B-architecture random-init Q8_0 decode, TP = world,
    KV caches pre-filled to 4096 positions, batch 1 (attention in the declared split order, S = 16) and batch 32
    (one-pass order), `steps` greedy steps from a captured graph.  With world > 1 rank 0 then re-runs the same
    tokens at TP = 1 and reports how often it chooses the same next token and the largest logit gap."""
    from llamatov_b200 import measure
    cfg = measure.tp_arch_cfg("llama-3-8b")
    out = {"world": world, "arch": "llama-3-8b", "context": 4096, "steps": steps}
    for B, split in ((1, 16), (32, 0)):
        r = measure.tp_decode_case(cfg, "llama-3-8b", rank, world, B, 4096, steps, 3, comm="p2p", attn_split=split,
                                   check_world1=world > 1, exact_split=True)
        m = r["token_match_vs_world1"] or {}
        out[f"batch{B}"] = {"tok_s": r["value"], "ms_per_step": r["ms_per_step"], "frac_of_ranks_x_hbm_peak": r["roofline"]["frac"],
                            "allreduce_share": r["allreduce_share"], "launches_per_step": r["config"]["launches_per_step"],
                            "token_match_vs_world1": m.get("same_next_token_given_same_history"),
                            "max_abs_logit_vs_world1": m.get("largest_logit_gap_where_different"),
                            "exact_down_split": r["config"]["exact_down_split"], "attention_order": r["config"]["attention_order"],
                            "device_status": r["device_status"]}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--repeats", type=int, default=5, help="timed regions of --steps steps each; the median is reported")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-tp", action="store_true", help="skip the tensor-parallel leg (the `tp` object)")
    ap.add_argument("--tp-steps", type=int, default=32)
    ap.add_argument("--config0", action="store_true", help="the single-GEMV case (BASELINE config 0) instead of decode")
    ap.add_argument("--step-mode", default=None, choices=["pdl", "persistent", "per-op"],
                    help="how the captured decode step is built (default: the engine's default)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.config0:
        if rank == 0:
            run_config0(args)
        return
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist
    from llamatov_b200 import _lib, dev_residency as dr, synth
    torch.cuda.set_device(local)
    if world > 1:
        import datetime
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=180))

    model = synth.make_model(ARCH, seed=0)
    mc = model["cfg"]
    V, E = mc["vocab"], mc["n_embd"]
    prompt = np.random.default_rng(0).integers(0, V, size=PROMPT_LEN).tolist()
    dr.reset_engine_state(); dr.apply_production_profile()
    if args.step_mode is not None:
        dr._FUSED_STEP = False if args.step_mode == "per-op" else args.step_mode
    # room in the KV caches for the prompt, the warm-up and the timed steps (the engine's default of 256
    # positions holds the default run; a longer run gets longer caches)
    need = PROMPT_LEN + args.steps + args.warmup + 8
    if need > dr._KV_MAX_SEQ:
        dr._KV_MAX_SEQ = ((need + 63) // 64) * 64
    w, cfg = synth.reference_weights(model)

    # ---- prompt (eager, token by token, as the reference does) + capture
    kv = [None] * cfg["n_layers"]
    gr = dr.GraphRunner(w, cfg, kv)
    logits = gr.seed(torch.tensor(prompt), torch.arange(PROMPT_LEN))
    first = int(np.argmax(logits.reshape(-1).numpy()))
    gr.capture(torch.tensor([first]), torch.tensor([PROMPT_LEN]))
    K, W = args.steps, args.warmup
    max_new = dr._KV_MAX_SEQ - PROMPT_LEN

    def reset_cache():
        """Back to the end of the prompt, so that every timed run decodes the same positions."""
        for c in kv:
            c.length = PROMPT_LEN
            c._len.fill_(PROMPT_LEN)
        torch.cuda.synchronize()

    from llamatov_b200 import replicas

    def barrier():
        torch.cuda.synchronize()
        replicas.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        return replicas.max_over_ranks(ms, device="cuda")

    if K + W > max_new:
        raise SystemExit(f"steps+warmup = {K + W} exceeds the KV capacity left after the prompt ({max_new})")

    R = max(1, args.repeats)
    # ---- e2e: the reference-facing call, host buffers, copies inside the timed region
    sampler = ClockSampler(local); sampler.start()
    e2e_runs, e2e_tokens = [], []
    for r in range(R):
        reset_cache()
        tok = first
        for _ in range(W):
            tok = gr.replay_token(tok)
        barrier()
        t0 = time.perf_counter()
        e2e_tokens = []
        for _ in range(K):
            tok = gr.replay_token(tok)
            e2e_tokens.append(tok)
        barrier()
        e2e_runs.append(max_over_ranks((time.perf_counter() - t0) * 1000.0))
    e2e_ms = float(np.median(e2e_runs))
    e2e_launches = (gr.launches_per_token + 2) * K

    # ---- value: device-resident token loop, CUDA events on the replay stream
    reset_cache()
    gr.capture_device_loop(first)
    dev_runs, dev_tokens = [], []
    for r in range(R):
        reset_cache()
        gr.reset_device_loop(first)
        gr.replay_device(W)
        barrier()
        ev0 = torch.cuda.Event(enable_timing=True); ev1 = torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(gr.stream):
            ev0.record()
        gr.replay_device(K)
        with torch.cuda.stream(gr.stream):
            ev1.record()
        barrier()
        dev_runs.append(max_over_ranks(ev0.elapsed_time(ev1)))
        dev_tokens = gr.device_tokens()[W:W + K]
    dev_ms = float(np.median(dev_runs))
    clocks = sampler.stop()
    status = _lib.device_status()
    tokens_match = (dev_tokens == e2e_tokens)

    # ---- roofline.  The step is one chain of kernels whose job is to stream every weight once:
    # algorithmic bytes per token = 34 B per 32 weights of every matrix + the fp32 KV rows read
    # once per KV head (at the middle position of the timed run), over the device time per token
    # measured above with CUDA events on the replay stream.
    nq = mc["n_head"] * mc["hd"]; nk = mc["n_head_kv"] * mc["hd"]
    weight_bytes = sum(M_ * (K_ // 32) * 34 * n_ for (M_, K_, n_) in gemv_shapes(mc))
    mid_len = PROMPT_LEN + W + K // 2
    kv_bytes = mc["n_layers"] * 2 * mid_len * nk * 4
    step_bytes = weight_bytes + kv_bytes
    peak, peak_src = _peaks()
    achieved = step_bytes / (dev_ms / K * 1e-3) / 1e9
    step_mode = getattr(gr, "_step_dev", None).mode if getattr(gr, "_step_dev", None) is not None else "per-op"
    # the one launch of the chain that is bandwidth-bound by itself: the LM-head GEMV, timed alone
    # (its 145 MB exceed L2, so every launch streams from HBM)
    dWq, dWd, N_, K_ = dr._weights(dr._lm_head(w))
    xq = torch.randint(-127, 128, (K_,), dtype=torch.int8, device="cuda")
    xd = torch.full((K_ // 32,), 0x2000, dtype=torch.int16, device="cuda")
    ybuf = torch.empty(N_, dtype=torch.float32, device="cuda")
    s2 = torch.cuda.Stream()
    torch.cuda.synchronize()
    with torch.cuda.stream(s2):
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        for _ in range(W):
            _lib.call("lt_q8_gemv", dWq, dWd, xq.data_ptr(), xd.data_ptr(), None, ybuf.data_ptr(), N_, K_, 1, st)
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            _lib.call("lt_q8_gemv", dWq, dWd, xq.data_ptr(), xd.data_ptr(), None, ybuf.data_ptr(), N_, K_, 1, st)
        e1.record()
    torch.cuda.synchronize()
    lm_us = 1000.0 * e0.elapsed_time(e1) / 20
    lm_gbs = gemv_bytes(N_, K_) / (lm_us * 1e-6) / 1e9
    # what this GPU's memory delivers right now: a device-to-device copy of 1 GiB (read + write counted), the same
    # kind of figure as the measured peak; a value far below the peak means the roofline fraction above is that
    # of a slowed GPU, not of the kernel
    src = torch.empty(1 << 30, dtype=torch.uint8, device="cuda"); dst = torch.empty_like(src)
    for _ in range(2):
        dst.copy_(src)
    c0 = torch.cuda.Event(enable_timing=True); c1 = torch.cuda.Event(enable_timing=True)
    c0.record()
    for _ in range(5):
        dst.copy_(src)
    c1.record(); torch.cuda.synchronize()
    copy_gbs = 5 * 2 * (1 << 30) / (c0.elapsed_time(c1) * 1e-3) / 1e9
    del src, dst
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": NCU_TRAFFIC.get(step_mode),
                "kernel": "decode step = %d launches per token (%s)" % (
                    gr.launches_per_step, "k_fused_gemv, k_fused_gateup, k_fused_attn, k_fused_lmhead, k_fused_argmax"
                    if step_mode == "pdl" else ("lt::k_decode_step, one cooperative launch" if step_mode == "persistent"
                                                else "per-op kernels")),
                "traffic_source": "ncu capture of this command (dram__bytes_read.sum + dram__bytes_write.sum of one "
                                  "token's launches), not measured in this run" if NCU_TRAFFIC.get(step_mode) else None,
                "algorithmic_bytes_per_launch": step_bytes / max(1, gr.launches_per_step),
                "algorithmic_bytes_per_token": step_bytes,
                "us_per_token": 1000.0 * dev_ms / K,
                "peak_source": peak_src,
                "hbm_copy_live": {"gbs": copy_gbs, "frac_of_peak": copy_gbs / peak,
                                  "what": "1 GiB device-to-device copy timed in this run (read + write bytes)"},
                "lm_head_gemv_alone": {"kernel": "lt::k_q8_gemv1<4,1>", "shape": [N_, K_], "us": lm_us,
                                       "achieved": lm_gbs, "frac": lm_gbs / peak}}

    # where the hand-over workspaces of the one-kernel step were put (chosen by timing a few steps per candidate
    # position before the graphs were captured; not part of the timed regions)
    placement = None
    pu = getattr(getattr(gr, "_step_dev", None), "placement_us", None)
    if pu:
        placement = {"chosen": list(gr._step_dev.placement), "tried": len(pu), "us_per_step_best": round(min(u for _, u in pu), 1),
                     "us_per_step_worst": round(max(u for _, u in pu), 1), "us_per_step_first": round(pu[0][1], 1)}
    value = world * K / (dev_ms * 1e-3)
    e2e_val = world * K / (e2e_ms * 1e-3)
    out = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
           "repeats": R, "value_min": world * K / (max(dev_runs) * 1e-3), "value_max": world * K / (min(dev_runs) * 1e-3),
           "ms_per_step": dev_ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": "int8*int8->int32, fp32 accumulate", "data": "synthetic",
           "config": {"workload": f"{ARCH} Q8_0 decode, batch 1, {PROMPT_LEN}-token prompt, {K} greedy steps",
                      "parallelism": "replicas only" if world > 1 else "1 GPU",
                      "l2": "inputs larger than L2 (525 MB of weights streamed per token vs 126 MB L2)",
                      "step_mode": step_mode, "timing": f"median of {R} timed regions of {K} steps",
                      "tokens_device_loop_equal_host_loop": tokens_match, "device_status": sorted(status),
                      "workspace_placement": placement},
           "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": gr.input_bytes_per_replay(), "d2h_bytes_per_step": 4,
                   "ms_per_step": e2e_ms / K, "value_min": world * K / (max(e2e_runs) * 1e-3),
                   "value_max": world * K / (min(e2e_runs) * 1e-3)},
           "gpu_launches": int(gr.launches_per_step * K),
           "gpu_launches_e2e": int(e2e_launches),
           "clocks": clocks, "roofline": roofline}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_decode_baseline(model, prompt)
    # ---- the tensor-parallel leg.  A failure or a stall here must not cost the line above: a watchdog prints
    # the line without the leg's numbers and ends the process.
    printed = threading.Event()

    def emit(tp_obj):
        if printed.is_set():
            return
        printed.set()
        out["tp"] = tp_obj
        if rank == 0:
            print(json.dumps(out), flush=True)

    if args.no_tp:
        emit(None)
    else:
        def give_up():
            emit({"error": "the tensor-parallel leg did not finish within its time limit"})
            sys.stdout.flush()
            os._exit(0)
        dog = threading.Timer(420.0, give_up); dog.daemon = True; dog.start()
        try:
            # free the 0.5B engine first: the leg builds an 8B model
            del gr, kv, w, model
            dr.reset_engine_state()
            torch.cuda.empty_cache()
            tp_obj = run_tp_leg(rank, world, args.tp_steps)
        except Exception as e:      # noqa: BLE001 -- the headline must survive anything the leg does
            tp_obj = {"error": f"{type(e).__name__}: {e}"[:400]}
        dog.cancel()
        emit(tp_obj)
    sys.stdout.flush()
    if world > 1:
        # no interpreter teardown: a process group being destroyed can wait on a peer that has already gone
        os._exit(0)


if __name__ == "__main__":
    main()
