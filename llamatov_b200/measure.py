"""Measurements beside the headline decode bench: prompt prefill and the GEMV / skinny-GEMM sweep.

  python -m llamatov_b200.measure prefill [--tokens 2048] [--batch 1 8] [--arch qwen2.5-0.5b]
  python -m llamatov_b200.measure gemv-sweep [--batch 1 4 16 64]
  python -m llamatov_b200.measure gemm -m 4864 -k 896 -t 2048 [--variant 1]
  python -m llamatov_b200.measure decode-trace [--cta N]
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
      -m llamatov_b200.measure tp-decode [--batch 1 32] [--ctx 4096] [--steps 128] [--check-world1]

Every line printed is one JSON object.  All timing is CUDA events on the launching stream after
warm-up; inputs are synthetic (llamatov_b200.synth), seeded.
"""
import argparse
import ctypes
import json
import os
import sys

import numpy as np
import torch

from . import _lib, synth
from . import dev_residency as dr
from . import prefill as pf

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SWEEP_SHAPES = [(896, 896), (128, 896), (4864, 896), (896, 4864), (151936, 896), (4096, 4096), (14336, 4096),
                (4096, 14336), (128256, 4096)]


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        j = json.load(open(p))
        return float(j["hbm_gbs"]), float(j.get("bf16_tflops", 0.0)), "measured"
    return 6650.0, 1590.0, "fallback"


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _event_ms(fn, reps):
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(reps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def gemv_bytes(M, K, T):
    """Algorithmic bytes of one launch: 34 B per 32 weights + T * (4K + 4M)."""
    return M * (K // 32) * 34 + T * (4 * K + 4 * M)


def run_prefill(args):
    hbm, _tf, src = peaks()
    model = synth.make_model(args.arch, seed=0)
    mc = model["cfg"]
    w, cfg = synth.reference_weights(model)
    T = args.tokens
    # int8 multiply-accumulates of the Q8_0 GEMMs per prompt token
    E, F = mc["n_embd"], mc["n_ffn"]
    nq, nk = mc["n_head"] * mc["hd"], mc["n_head_kv"] * mc["hd"]
    macs = mc["n_layers"] * ((nq + 2 * nk) * E + E * nq + 2 * F * E + E * F)
    for B in args.batch:
        dr.reset_engine_state(); dr.apply_production_profile()
        dr._KV_MAX_SEQ = T
        rng = np.random.default_rng(0)
        toks = torch.from_numpy(rng.integers(0, mc["vocab"], size=(B, T)).astype(np.int64))
        times = []
        for it in range(args.warmup + args.steps):
            kvs = [[None] * cfg["n_layers"] for _ in range(B)]
            torch.cuda.synchronize()
            e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
            n0 = _lib.launch_count()
            e0.record()
            pf.prefill_resident(w, cfg, toks, kvs, want_logits=True)
            e1.record(); torch.cuda.synchronize()
            if it >= args.warmup:
                times.append(e0.elapsed_time(e1))
            launches = _lib.launch_count() - n0
            for kv in kvs:
                for c in kv:
                    c.free()
            del kvs
        ms = float(np.median(times))
        print(json.dumps({
            "metric": "prefill tok/s (Q8_0, batched pass)", "value": B * T / (ms * 1e-3), "unit": "tok/s",
            "ms_per_prompt_batch": ms, "config": {"workload": f"{args.arch} Q8_0 prefill, {T}-token prompt, batch {B}",
                                                  "rows_per_pass": B * T},
            "gpu_launches": launches, "steps": args.steps, "warmup": args.warmup,
            "int8_tmacs_per_s": macs * B * T / (ms * 1e-3) / 1e12,
            "device_status": sorted(_lib.device_status()), "data": "synthetic", "peak_source": src}), flush=True)


def run_gemv_sweep(args):
    hbm, _tf, src = peaks()
    shapes = SWEEP_SHAPES
    L2_BYTES = 126e6
    for (M, K) in shapes:
        nb = K // 32
        wbytes = M * nb * 34
        # steady state: enough distinct copies of the matrix that consecutive launches cannot hit L2 (the copies
        # together are 2.5 x L2 at least, however small the matrix is)
        R = int(max(2, np.ceil(2.5 * L2_BYTES / wbytes)))
        Wq = torch.randint(-127, 128, (R, M * K), dtype=torch.int8, device="cuda")
        Wd = (torch.rand((R, M * nb), device="cuda") * 0.02).to(torch.float16).view(torch.int16)
        for T in args.batch:
            xq = torch.randint(-127, 128, (T * K,), dtype=torch.int8, device="cuda")
            xd = (torch.rand((T * nb,), device="cuda") * 0.05).to(torch.float16).view(torch.int16)
            y = torch.empty(T * M, dtype=torch.float32, device="cuda")

            def run(i):
                r = i % R
                _lib.call("lt_q8_gemv", Wq[r].data_ptr(), Wd[r].data_ptr(), xq.data_ptr(), xd.data_ptr(), None,
                          y.data_ptr(), M, K, T, _stream())
            for i in range(max(3, R)):
                run(i)
            torch.cuda.synchronize()
            # steady state: a captured chain of launches over the rotating copies, so that the host's
            # launch rate does not enter (small shapes run for ~2 us)
            chain = R if R >= 256 else max(R, (int(min(256, 2e9 // max(wbytes, 1))) // R) * R)
            side = torch.cuda.Stream()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for i in range(chain):
                    run(i)
            with torch.cuda.stream(side):
                for _ in range(2):
                    g.replay()
                side.synchronize()
                ms = _event_ms(lambda i: g.replay(), 5) / chain
            # one launch alone with a cold L2: the flush (a write larger than L2) is queued first, the
            # events and the launch behind it, so the host's launch latency is hidden behind the flush
            flush = torch.empty(int(2 * L2_BYTES), dtype=torch.uint8, device="cuda")
            cold = []
            for i in range(5):
                e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
                flush.fill_(i)
                e0.record(); run(i); e1.record()
                torch.cuda.synchronize()
                cold.append(e0.elapsed_time(e1))
            del flush
            # grouped form: ONE launch over the R distinct matrices (they lie back to back, so the launch is the
            # GEMV of the stacked [R*M, K] matrix): what the kernel sustains on this row length when launch
            # latency and the ramp / tail of a tiny grid do not enter
            yg = torch.empty(T * R * M, dtype=torch.float32, device="cuda")

            def run_grouped(i):
                _lib.call("lt_q8_gemv", Wq.data_ptr(), Wd.data_ptr(), xq.data_ptr(), xd.data_ptr(), None,
                          yg.data_ptr(), R * M, K, T, _stream())
            for i in range(3):
                run_grouped(i)
            torch.cuda.synchronize()
            gms = _event_ms(run_grouped, 5) / R
            del yg
            b = gemv_bytes(M, K, T)
            print(json.dumps({"M": M, "K": K, "batch": T, "algorithmic_bytes": b,
                              "grouped_us_per_matrix": gms * 1e3, "grouped_GBs": b / (gms * 1e-3) / 1e9,
                              "grouped_frac_of_hbm": b / (gms * 1e-3) / 1e9 / hbm,
                              "steady_us": ms * 1e3, "steady_GBs": b / (ms * 1e-3) / 1e9,
                              "steady_frac_of_hbm": b / (ms * 1e-3) / 1e9 / hbm,
                              "alone_cold_us": float(np.median(cold)) * 1e3,
                              "alone_cold_frac_of_hbm": b / (float(np.median(cold)) * 1e-3) / 1e9 / hbm,
                              "copies_in_rotation": R, "peak_GBs": hbm, "peak_source": src}), flush=True)
        del Wq, Wd
    print(json.dumps({"device_status": sorted(_lib.device_status())}))


def run_gemm(args):
    """One Q8_0 GEMM shape through lt_q8_gemm_tc (or lt_q8_gemv with --variant -1), resident random data."""
    hbm, _tf, src = peaks()
    M, K, T = args.m, args.k, args.t
    nb = K // 32
    Wq = torch.randint(-127, 128, (M * K,), dtype=torch.int8, device="cuda")
    Wd = (torch.rand((M * nb,), device="cuda") * 0.02).to(torch.float16).view(torch.int16)
    xq = torch.randint(-127, 128, (T * K,), dtype=torch.int8, device="cuda")
    xd = (torch.rand((T * nb,), device="cuda") * 0.05).to(torch.float16).view(torch.int16)
    y = torch.empty(T * M, dtype=torch.float32, device="cuda")

    def run(i):
        if args.variant < 0:
            _lib.call("lt_q8_gemv", Wq.data_ptr(), Wd.data_ptr(), xq.data_ptr(), xd.data_ptr(), None, y.data_ptr(),
                      M, K, T, _stream())
        else:
            _lib.call("lt_q8_gemm_tc", Wq.data_ptr(), Wd.data_ptr(), xq.data_ptr(), xd.data_ptr(), None, 0,
                      y.data_ptr(), M, K, T, args.variant, _stream())
    for i in range(args.warmup):
        run(i)
    torch.cuda.synchronize()
    ms = _event_ms(run, args.steps)
    b = gemv_bytes(M, K, T)
    print(json.dumps({"M": M, "K": K, "T": T, "variant": args.variant, "us": ms * 1e3,
                      "output_blocks_per_s": M * nb * T / (ms * 1e-3), "int8_tmacs_per_s": M * K * T / (ms * 1e-3) / 1e12,
                      "algorithmic_GBs": b / (ms * 1e-3) / 1e9, "frac_of_hbm": b / (ms * 1e-3) / 1e9 / hbm,
                      "device_status": sorted(_lib.device_status()), "peak_source": src}))


TRACE_IDS = {1: "kernel entry", 11: "attention CTA: layer input x in shared memory", 111: "... RMSNorm + quantiser done",
             12: "... q|k rows folded", 13: "... rope, K append, scores done", 14: "... softmax, V fold, head output published",
             20: "GEMV CTA: phase prepared (weight stages awaited, addresses, operands)",
             21: "phase 0: x arrived", 22: "phase 1: attention output arrived", 23: "phase 2: x1 arrived",
             24: "phase 3: silu*up arrived", 25: "phase 0 done (v rows stored) / LM head done", 26: "phase 1 done (x1 stored)",
             27: "phase 2 done (silu*up published)", 28: "phase 3 done (x stored)", 32: "LM head: CTA's rows done",
             99: "end (the last CTA: all partial argmax results collected)"}


def run_decode_trace(args):
    """SM-clock stamps inside the one-kernel decode step (lt_decode_step, trace pointer set): for CTA 0 (an
    attention CTA) and one GEMV CTA (--cta, default the last), the mean / min / max time from the previous
    stamp to each stamp over the layers.  One JSON line per traced CTA."""
    if args.cta:
        os.environ["LLAMATOV_TRACE_CTA"] = str(args.cta)
    if args.layer >= 0:
        os.environ["LLAMATOV_TRACE_LAYER"] = str(args.layer)
    dr._FUSED_STEP = "persistent"
    m = synth.make_model(args.arch, seed=0)
    w, cfg = synth.reference_weights(m)
    dr.reset_engine_state(); dr.apply_production_profile()
    kv = [None] * cfg["n_layers"]
    gr = dr.GraphRunner(w, cfg, kv)
    prompt = np.random.default_rng(0).integers(0, m["cfg"]["vocab"], size=32).tolist()
    lg = gr.seed(torch.tensor(prompt), torch.arange(32))
    first = int(np.argmax(lg.reshape(-1).numpy()))
    tokd = torch.tensor([first], dtype=torch.int32, device="cuda")
    st = dr.FusedDecodeStep(w, cfg, kv, tok_ptr=tokd.data_ptr())
    if st.mode != "persistent":
        raise SystemExit("the one-kernel step does not support this architecture")
    st.tune_placement()          # the workspaces where the engine would put them
    n = st.enable_trace()
    for _ in range(4):
        st.launch()
    torch.cuda.synchronize()
    st.trace.zero_()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record(); st.launch(); e1.record(); torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    try:
        mhz = float(torch.cuda.clock_rate())        # SM clock now, MHz (NVML)
    except Exception:
        mhz = 1965.0
    if args.layer >= 0:
        # one layer on the global timer: [cta][arrival of phase 0..3, end of phase 0..3], ns
        G = _lib.lib().lt_decode_num_ctas()
        nh = m["cfg"]["n_head"]
        a = st.trace.cpu().numpy().reshape(-1)[4 * n - 8 * G:].reshape(G, 8).astype(np.int64)[nh:]      # the GEMV CTAs
        a = (a - a[:, 0].min()) / 1000.0
        names = ["x arrived", "attention output arrived", "x1 arrived", "silu*up arrived", "phase 0 done (v rows stored)",
                 "phase 1 done (x1 stored)", "phase 2 done (silu*up published)", "phase 3 done (next x stored)"]
        nblk = m["cfg"]["n_ffn"] // 32
        two = [c for c in range(G - nh) if (nblk * (c + 1)) // (G - nh) - (nblk * c) // (G - nh) >= 2]
        rows = {names[j]: {"earliest": round(float(a[:, j].min()), 2), "median": round(float(np.median(a[:, j])), 2),
                           "latest": round(float(a[:, j].max()), 2)} for j in (0, 4, 1, 5, 2, 6, 3, 7)}
        if two:
            rows["phase 2 done, CTAs with two or more gate|up blocks"] = {"median": round(float(np.median(a[two, 6])), 2),
                                                                          "latest": round(float(a[two, 6].max()), 2)}
        print(json.dumps({"layer": args.layer, "gemv_ctas": G - nh, "us_from_first_arrival_of_x": rows}), flush=True)
    tr = st.trace.cpu().numpy().reshape(2, n, 2)
    for c in range(2):
        tt = tr[c]
        k = int(np.argmax(tt[:, 1] == 0)) if (tt[:, 1] == 0).any() else n
        ids, clk = tt[:k, 0], tt[:k, 1]
        rows = {}
        for i in range(1, k):
            rows.setdefault(int(ids[i]), []).append((clk[i] - clk[i - 1]) / mhz)
        print(json.dumps({"cta": "0 (attention, head 0)" if c == 0 else f"{args.cta or 'last'} (GEMV)", "launch_ms_traced": ms,
                          "sm_mhz_assumed": mhz, "total_us": float((clk[-1] - clk[0]) / mhz),
                          "us_since_previous_stamp": {TRACE_IDS.get(i, str(i)): {"n": len(v), "mean": round(float(np.mean(v)), 2),
                                                                                 "min": round(float(np.min(v)), 2),
                                                                                 "max": round(float(np.max(v)), 2)}
                                                      for i, v in sorted(rows.items())},
                          "device_status": sorted(_lib.device_status())}), flush=True)


def tp_arch_cfg(arch, layers=0):
    a = synth.ARCHS[arch]
    cfg = dict(n_layers=a["n_layers"], n_head=a["n_head"], n_head_kv=a["n_head_kv"], n_embd=a["n_embd"],
               rope_theta=a["rope_theta"], norm_eps=a["norm_eps"], hd=a["hd"], n_ffn=a["n_ffn"], vocab=a["vocab"],
               tied=a["tied"])
    if layers:
        cfg["n_layers"] = layers
    return cfg


def tp_decode_case(cfg, arch, rank, world, B, ctx, steps, warmup, comm="p2p", attn_split=0, chained=False,
                   fused_allreduce=True, check_world1=False, exact_split=True):
    """One tensor-parallel decode measurement: B sequences, KV caches pre-filled to `ctx` positions,
    `steps` greedy steps from a captured graph, CUDA events, max over ranks.  Every rank of the
    (already initialised) process group must call it; every rank gets the result dict."""
    import torch.distributed as dist
    from . import tp
    hbm, _tf, src = peaks()
    E, F, V, L = cfg["n_embd"], cfg["n_ffn"], cfg["vocab"], cfg["n_layers"]
    nq, nk = cfg["n_head"] * cfg["hd"], cfg["n_head_kv"] * cfg["hd"]
    wbytes = (L * ((nq + 2 * nk) * E + E * nq + 2 * F * E + E * F) + V * E) // 32 * 34
    max_seq = ctx + steps + warmup + 8
    dec = tp.TPDecoder(cfg, rank=rank, world=world, batch=B, max_seq=max_seq, seed=0, comm=comm,
                       attn_split=attn_split, chained=bool(chained), fused_allreduce=bool(fused_allreduce),
                       exact_split=bool(exact_split))
    dec.fill_cache(ctx, seed=1)
    start = np.random.default_rng(0).integers(0, V, size=B)
    dec.set_tokens(start)
    dec.capture()                               # one warm-up step inside
    warm = [dec.tok.clone()]
    for _ in range(max(0, warmup - 1)):
        dec.graph.replay()
        warm.append(dec.tok.clone())
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    toks = []
    for _ in range(steps):
        dec.graph.replay()
        toks.append(dec.tok.clone())
    e1.record(); torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    toks = torch.stack(toks).cpu().numpy()
    t = torch.tensor([ms], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    # the all-reduces of one step alone, back to back (2 per layer, [B, E] fp32)
    ar_ms = 0.0
    if world > 1:
        buf = torch.zeros((B, E), device="cuda"); buf2 = torch.zeros((B, E), device="cuda")
        side = torch.cuda.Stream()

        def one():
            if dec.comm is not None:
                dec.comm.allreduce_add(buf, None, buf2, B * E)
            else:
                dist.all_reduce(buf)
        with torch.cuda.stream(side):
            one()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for _ in range(2 * L):
                one()
        g.replay(); torch.cuda.synchronize()
        dist.barrier()
        ar_ms = _event_ms(lambda i: g.replay(), 10)
        t = torch.tensor([ar_ms], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX); ar_ms = float(t.item())
    status = sorted(_lib.device_status())
    launches = dec.launches_per_step
    exact_used = bool(dec.exact)
    match = None
    if check_world1 and world > 1:
        # world 1 on rank 0's GPU, teacher-forced with the sharded run's tokens: does it choose the same
        # next token from the same history, and how far apart are its logits from the sharded run's choice
        dec.close()
        del dec
        torch.cuda.empty_cache()
        if rank == 0:
            ref = tp.TPDecoder(cfg, rank=0, world=1, batch=B, max_seq=max_seq, seed=0, attn_split=attn_split)
            ref.fill_cache(ctx, seed=1)
            ref.set_tokens(start)
            warm_h = torch.stack(warm).cpu().numpy()
            allt = np.concatenate([warm_h, toks], axis=0)      # every token the sharded run produced, warm-up included
            agree, worst = 0, 0.0
            for sidx in range(allt.shape[0]):
                ref.step()
                rt = ref.tok.cpu().numpy()
                lg = ref.logits
                for b in range(B):
                    if rt[b] == allt[sidx, b]:
                        agree += 1
                    else:
                        worst = max(worst, float(lg[b, int(rt[b])] - lg[b, int(allt[sidx, b])]))
                ref.set_tokens(allt[sidx])
            match = {"same_next_token_given_same_history": agree / (allt.shape[0] * B),
                     "largest_logit_gap_where_different": worst}
            ref.close()
            del ref
        dist.barrier()
    else:
        dec.close()
        del dec
    torch.cuda.empty_cache()
    step_ms = ms / steps
    kv_bytes = B * L * 2 * (ctx + steps // 2) * nk * 4
    step_bytes = wbytes + kv_bytes
    return {
        "metric": "decode tok/s (Q8_0, tensor-parallel)", "value": B * steps / (ms * 1e-3), "unit": "tok/s",
        "n_gpus": world, "ms_per_step": step_ms, "steps": steps, "warmup": warmup,
        "config": {"workload": f"{arch} Q8_0 decode, batch {B}, context {ctx}, TP={world}",
                   "layers": L, "launches_per_step": launches, "comm": comm if world > 1 else None,
                   "chained_launches": bool(chained),
                   "allreduce_in_gemv": bool(fused_allreduce) and world > 1 and comm == "p2p" and B == 1,
                   "exact_down_split": exact_used,
                   "attention_order": f"attn_decode_split, S={attn_split}" if attn_split else "one-pass (production)"},
        "roofline": {"bound": "hbm", "algorithmic_bytes_per_step": step_bytes,
                     "achieved": step_bytes / (step_ms * 1e-3) / 1e9, "peak": hbm * world, "unit": "GB/s",
                     "frac": step_bytes / (step_ms * 1e-3) / 1e9 / (hbm * world), "peak_source": src},
        "allreduce_ms_per_step_alone": ar_ms, "allreduce_share": ar_ms / step_ms if step_ms else None,
        "token_match_vs_world1": match, "first_tokens": toks[:4, 0].tolist(),
        "device_status": status, "data": "synthetic"}


def run_tp_decode(args):
    """Llama-3-8B-architecture (or --arch) random-init Q8_0 decode, tensor-parallel over the ranks this
    program was launched with (torch.distributed.run; a plain launch is world 1)."""
    import datetime
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1")); rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local),
                                timeout=datetime.timedelta(seconds=120))
    cfg = tp_arch_cfg(args.arch, args.layers)
    for B in args.batch:
        out = tp_decode_case(cfg, args.arch, rank, world, B, args.ctx, args.steps, args.warmup, comm=args.comm,
                             attn_split=args.attn_split, chained=args.chained, fused_allreduce=args.fused_allreduce,
                             check_world1=args.check_world1, exact_split=args.exact_split)
        if rank == 0:
            print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0)


def main(argv=None):
    ap = argparse.ArgumentParser(prog="llamatov_b200.measure")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("prefill")
    p.add_argument("--arch", default="qwen2.5-0.5b")
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--batch", type=int, nargs="+", default=[1, 8])
    p.add_argument("--steps", type=int, default=3)
    p.add_argument("--warmup", type=int, default=1)
    g = sub.add_parser("gemv-sweep")
    g.add_argument("--batch", type=int, nargs="+", default=[1, 4, 16, 64])
    m = sub.add_parser("gemm")
    m.add_argument("-m", type=int, required=True); m.add_argument("-k", type=int, required=True)
    m.add_argument("-t", type=int, required=True)
    m.add_argument("--variant", type=int, default=0, help="lt_q8_gemm_tc variant; -1 = lt_q8_gemv dispatch")
    m.add_argument("--steps", type=int, default=2); m.add_argument("--warmup", type=int, default=1)
    d = sub.add_parser("decode-trace")
    d.add_argument("--arch", default="qwen2.5-0.5b")
    d.add_argument("--cta", type=int, default=0, help="index of the traced GEMV CTA (0 = the last CTA)")
    d.add_argument("--layer", type=int, default=-1,
                   help="also print the timeline of this layer on the global timer: every GEMV CTA's arrival and end of each phase")
    t = sub.add_parser("tp-decode")
    t.add_argument("--arch", default="llama-3-8b")
    t.add_argument("--batch", type=int, nargs="+", default=[1, 32])
    t.add_argument("--ctx", type=int, default=4096)
    t.add_argument("--steps", type=int, default=128)
    t.add_argument("--warmup", type=int, default=3)
    t.add_argument("--layers", type=int, default=0, help="fewer layers than the architecture (smoke runs)")
    t.add_argument("--comm", default="p2p", choices=["p2p", "nccl"])
    t.add_argument("--attn-split", type=int, default=0,
                   help="S > 0: decode attention in the reference's declared split order with S ranges; 0: one-pass order")
    t.add_argument("--fused-allreduce", type=int, default=1,
                   help="comm p2p, batch 1: 1 = the row-split GEMVs exchange their partial rows themselves "
                        "(lt_q8_gemv_allreduce); 0 = GEMV, then lt_allreduce_add")
    t.add_argument("--chained", type=int, default=0,
                   help="1: one-sequence operators as chained launches (lt_set_chained_launch; measured slower inside "
                        "a captured graph); 0: ordinary launches")
    t.add_argument("--check-world1", action="store_true", help="rank 0 re-runs at world 1 and compares the tokens")
    t.add_argument("--exact-split", type=int, default=1,
                   help="1: down is split by dealing Q8_0 blocks round-robin (lane-exact partial folds, tree-ordered "
                        "sum: the bits of one GPU); 0: contiguous K ranges")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("llamatov_b200.measure needs a CUDA device (there is no CPU path)")
    if args.cmd == "prefill":
        run_prefill(args)
    elif args.cmd == "tp-decode":
        run_tp_decode(args)
    elif args.cmd == "gemm":
        run_gemm(args)
    elif args.cmd == "decode-trace":
        run_decode_trace(args)
    else:
        run_gemv_sweep(args)


if __name__ == "__main__":
    main()
