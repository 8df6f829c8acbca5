#!/usr/bin/env python
"""Headline benchmark: LLaMA-7B-shape greedy decode (random-init bf16, synthetic prompt) in tokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl reference]

A "step" is one decode step: one new token for each of the B sequences of the batch, every weight byte
of the model and every cached K/V byte read once.  With N > 1 (launched by torch.distributed.run, one
rank per GPU) the model is tensor-parallel over attention heads and FFN columns with one all-reduce per
attention block and one per FFN block; the total work is fixed (strong scaling).

Rank 0 prints ONE JSON line.  `value` is timed on the device with CUDA events around K replayed steps
(inputs resident in HBM); `e2e` is the same loop driven through the C-ABI entry points with the token
ids coming from pinned host memory and the next tokens read back every step; `roofline` is the
weight-streaming projection kernel timed alone against the measured HBM peak; `cpu_baseline` is the
CPU oracle timed on a bounded sample of the same per-token work.

`--impl reference` times the reference's own CPU code (the jasmine headers behind oracle/_ref) on a
bounded sample of the per-token work and extrapolates by multiply-accumulate count.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LLAMA7B = dict(n_layers=32, d_model=4096, n_heads=32, n_kv_heads=32, d_ffn=11008, vocab=32000)
PROMPT, GEN = 512, 128
SEED = 4


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ---- clocks ----------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx = float(r[1])
                for n, v in zip(names, r[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                pass
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


# ---- CPU legs (the only places that touch oracle/) ------------------------------------------------
def per_token_macs(ctx: int) -> int:
    c = LLAMA7B
    d, ffn, L = c["d_model"], c["d_ffn"], c["n_layers"]
    return L * (4 * d * d + 3 * d * ffn + 2 * ctx * d) + c["vocab"] * d


def cpu_port_baseline():
    """Times the CPU oracle (port) on a slice of one decoder layer for one token and extrapolates by MAC count."""
    sys.path.insert(0, str(ROOT / "tests"))
    import numpy as np
    import oracle_lib as ol
    d, rows, ctx = LLAMA7B["d_model"], 2048, 512
    cores = os.cpu_count() or 1
    W = ol.fill(rows * d, SEED, 1, 0, 0.0, 0.02, to_bf16=True).reshape(rows, d)
    x = ol.fill(d, SEED, 2, 0, 0.0, 1.0, to_bf16=True).reshape(1, d)
    kv = ol.fill(ctx * d, SEED, 3, 0, 0.0, 1.0, to_bf16=True).reshape(ctx, d)
    po = ol.port_oracle()
    po.linear(x, W, np.zeros(rows, np.float32))  # warm
    t0 = time.perf_counter()
    reps = 0
    while time.perf_counter() - t0 < 10.0:
        po.linear(x, W, np.zeros(rows, np.float32))
        ol.attention(x, kv, kv, 1, 32, 32, 128, False, exact_div=False)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    macs = rows * d + 2 * ctx * d
    tok_s = 1.0 / (dt * per_token_macs(PROMPT + GEN // 2) / macs)
    return {"value": tok_s, "unit": "tok/s", "cores": cores, "kind": "port",
            "sample": f"{rows}x{d} projection + one attention row over {ctx} cached tokens for 1 token, OpenMP over "
                      f"{cores} threads, ~10 s, extrapolated by multiply-accumulate count to the full model"}


def run_reference_arm(args):
    """The reference's own weight_net_t::forward / attention code on the host cores (bounded sample per step)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sys.path.insert(0, str(ROOT / "tests"))
    import numpy as np
    import oracle_lib as ol
    ref = ol.ref_oracle()
    kind = "reference"
    if ref is None:
        ref, kind = ol.port_oracle(), "port"
    d, rows = LLAMA7B["d_model"], 256
    cores = os.cpu_count() or 1
    W = ol.fill(rows * d, SEED, 1, 0, 0.0, 0.02, to_bf16=True).reshape(rows, d)
    x = ol.fill(d, SEED, 2, 0, 0.0, 1.0, to_bf16=True).reshape(1, d)
    b = np.zeros(rows, np.float32)

    def step():
        # the reference is single-threaded by construction: independent row slices are farmed over the cores
        ts = [threading.Thread(target=ref.linear, args=(x, W, b)) for _ in range(cores)]
        for t in ts:
            t.start()
        for t in ts:
            t.join()

    for _ in range(max(1, min(args.warmup, 3))):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    macs = cores * rows * d
    tok_s = 1.0 / (dt * per_token_macs(PROMPT + GEN // 2) / macs)
    sample = (f"projection-only sample (no attention, no norms, no per-token prefix recompute); per step: {cores} concurrent "
              f"weight_net_t::forward calls ({rows}x{d} rows each, 1 token) through the "
              f"{'jasmine headers (oracle/_ref)' if kind == 'reference' else 'CPU oracle port'}; tok/s extrapolated by "
              f"multiply-accumulate count to one token of the 7B model at context {PROMPT + GEN // 2}")
    line = {"impl": "reference", "metric": "llama7b_decode_tokens_per_s", "value": tok_s, "unit": "tok/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args, 1),
            "cpu_baseline": {"value": tok_s, "unit": "tok/s", "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def workload_config(args, n):
    return {"workload": f"llama7b_decode_b{args.batch}", "layers": 32, "d_model": 4096, "heads": "32x128", "d_ffn": 11008,
            "vocab": 32000, "batch": args.batch, "prompt_len": PROMPT, "generated": GEN,
            "parallelism": f"tp{n}", "exchange": ("nccl" if os.environ.get("JSM_TP_NCCL", "0") == "1" else "peer memory") if n > 1 else "none", "l2": "inputs larger than L2 (13.2 GB of weights per step)"}


# ---- kernel-level workloads: configurations 2, 3 and 4 of the baseline ------------------------------------
def run_kernel_workload(args, collect=False):
    """One JSON line per kernel; with collect=True the records are returned instead of printed."""
    records = []
    import torch
    import jasmine_b200 as jb
    torch.cuda.set_device(0)
    hbm, peak_kind = measured_peaks()
    p = ROOT / "MEASURED_PEAKS.json"
    tf_peak = float(json.loads(p.read_text())["bf16_tflops"]) if p.exists() else 1590.0
    K, W = max(args.steps, 1), max(args.warmup, 3)

    def timed(fn, sets=1):
        """Mean milliseconds per call over K calls; `sets` rotating input sets keep the operands out of L2.  The K calls
        are captured into one CUDA graph and replayed, so that the time between the events is device time and not the
        rate at which Python can issue calls of a few tens of microseconds."""
        for i in range(W):
            fn(i % sets)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for i in range(K):
                    fn(i % sets)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / K

    def emit(name, ms, bound, work, peak, unit, config):
        ach = work / (ms * 1e-3) / (1e9 if bound == "hbm" else 1e12)
        rec = ({"metric": name, "value": ach, "unit": unit, "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms,
                          "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "data": "synthetic", "config": config,
                          "roofline": {"bound": bound, "achieved": ach, "peak": peak, "unit": unit, "frac": ach / peak,
                                       "traffic": None, "peak_source": f"{peak_kind}"}})
        if collect:
            records.append(rec)
        else:
            print(json.dumps(rec), flush=True)

    L0, L1 = (jb.OP_LEAF, 0), (jb.OP_LEAF, 1)
    if args.workload == "expr":
        n, sets = 4096, 4  # 4 sets x 192 MiB of operands: every launch reads from HBM, not from the 126 MB L2
        A = [torch.empty(n, n, device="cuda") for _ in range(sets)]
        B = [torch.empty(n, n, device="cuda") for _ in range(sets)]
        Y = [torch.empty(n, n, device="cuda") for _ in range(sets)]
        for i in range(sets):
            jb.fill(A[i], 1, 2 * i, 0, 0.0, 1.0); jb.fill(B[i], 1, 2 * i + 1, 0, 0.0, 1.0)
        g = torch.empty(n, device="cuda"); b = torch.empty(n, device="cuda"); r = torch.empty(n, 1, device="cuda")
        jb.fill(g, 1, 100, 1, 0.5, 1.5); jb.fill(b, 1, 101, 0, 0.0, 0.1)
        axpb = [L0, (jb.OP_IMM, 0.125), (jb.OP_MUL,), L1, (jb.OP_ADD,)]
        cfg = {"workload": "expr_4096x4096_f32", "l2": f"{sets} rotating operand sets (768 MiB) > L2"}
        full = n * n * 4
        emit("hsoftmax(A*0.125+B)_GBps", timed(lambda i: jb.eval_rows(jb.ROWS_SOFTMAX, 1, axpb, [A[i], B[i]], Y[i]), sets), "hbm", 3 * full, hbm, "GB/s", cfg)
        emit("LayerNorm_rows(A+B)*g+b_GBps", timed(lambda i: jb.eval_rows(jb.ROWS_LAYERNORM, 1, [L0, L1, (jb.OP_ADD,)], [A[i], B[i]], Y[i], gain=g, bias=b, eps=1e-5), sets),
             "hbm", 3 * full + 2 * n * 4, hbm, "GB/s", cfg)
        emit("RMSNorm_rows(A)*g_GBps", timed(lambda i: jb.eval_rows(jb.ROWS_RMSNORM, 1, [L0], [A[i]], Y[i], gain=g, eps=1e-5), sets), "hbm", 2 * full + n * 4, hbm, "GB/s", cfg)
        emit("row_sum_GBps", timed(lambda i: jb.eval_rows(jb.ROWS_SUM, 1, [L0], [A[i]], r), sets), "hbm", full + n * 4, hbm, "GB/s", cfg)
        emit("row_max_GBps", timed(lambda i: jb.eval_rows(jb.ROWS_MAX, 1, [L0], [B[i]], r), sets), "hbm", full + n * 4, hbm, "GB/s", cfg)
        emit("elementwise_A*0.125+B_GBps", timed(lambda i: jb.eval_elementwise(axpb, [A[i], B[i]], Y[i]), sets), "hbm", 3 * full, hbm, "GB/s", cfg)
    elif args.workload == "gateup":
        # one SwiGLU gate/up projection of the 7B shape, alone: [2 x 11008, 4096] bf16 weights (180 MB) streamed once per
        # launch against B tokens; 4 rotating weight sets keep every launch out of L2
        d, ffn, Bt, sets = 4096, 11008, args.batch, 4
        Ws = [torch.empty(2 * ffn, d, device="cuda", dtype=torch.bfloat16) for _ in range(sets)]
        for i, w in enumerate(Ws):
            jb.fill(w, SEED, 9000 + i, 0, 0.0, 0.02)
        x = torch.empty(Bt, d, device="cuda", dtype=torch.bfloat16); jb.fill(x, SEED, 7000, 0, 0.0, 1.0)
        y = torch.empty(Bt, ffn, device="cuda", dtype=torch.bfloat16)
        cfg = {"workload": f"gate_up_projection_11008x4096_b{Bt}", "l2": f"{sets} rotating weight sets (720 MB) > L2"}
        work = 2 * ffn * d * 2 + Bt * d * 2 + Bt * ffn * 2

        def once(i):
            jb.check(jb.lib().jsm_linear_bf16(x.data_ptr(), Ws[i].data_ptr(), None, 3, None, y.data_ptr(), jb.BF16, Bt, ffn, d,
                                              jb.stream_ptr()))
        emit("gate_up_projection_GBps", timed(once, sets), "hbm", work, hbm, "GB/s", cfg)
        # the same projection over packed weights (contiguous 16 KB tiles, stream-K split over all SMs)
        Wp = [jb.linear_pack(w, ffn, paired=True) for w in Ws]

        def once_packed(i):
            jb.check(jb.lib().jsm_linear_bf16_packed(x.data_ptr(), Wp[i].data_ptr(), None, 3, None, y.data_ptr(), jb.BF16, Bt,
                                                     ffn, d, jb.stream_ptr()))
        once_packed(0)
        jb.check_device_errors()
        emit("gate_up_projection_packed_GBps", timed(once_packed, sets), "hbm", work, hbm, "GB/s", cfg)
    elif args.workload == "flash":
        batch, T, H, D = 4, 4096, 32, 128
        q = torch.empty(batch * T, H * D, device="cuda", dtype=torch.bfloat16)
        k = torch.empty_like(q); v = torch.empty_like(q); o = torch.empty_like(q)
        jb.fill(q, 2, 0, 0, 0.0, 1.0); jb.fill(k, 2, 1, 0, 0.0, 1.0); jb.fill(v, 2, 2, 0, 0.0, 1.0)
        table = jb.rope_table(1, D, 10000.0, T)
        pos = torch.arange(T, dtype=torch.int32, device="cuda").repeat(batch)
        qr, kr = torch.empty_like(q), torch.empty_like(k)
        flops = 4.0 * batch * H * T * T * D / 2  # causal convention: half of the S x S scores
        cfg = {"workload": "flash_prefill_b4_h32_s4096_d128_causal_bf16", "l2": "512 MiB of q, k, v, out > L2"}

        def attn_only(_):
            jb.attn_prefill(qr, kr, v, batch, H, H, D, causal=True, impl=2, out=o)

        def with_rope(_):
            jb.rope_apply_qk(q, k, table, D, H, H, positions=pos, q_out=qr, k_out=kr)
            jb.attn_prefill(qr, kr, v, batch, H, H, D, causal=True, impl=2, out=o)
        with_rope(0)
        jb.check_device_errors()  # a kernel that gave up on a wait must not be timed
        emit("flash_prefill_TFLOPs", timed(attn_only), "tensor", flops, tf_peak, "TFLOP/s", cfg)
        emit("flash_prefill_with_rope_TFLOPs", timed(with_rope), "tensor", flops, tf_peak, "TFLOP/s", cfg)
    else:
        sys.path.insert(0, str(ROOT))
        Hq, Hkv, D, n = 32, 8, 128, 64
        lens_t = torch.empty(n, dtype=torch.int32)
        jb.fill(lens_t, 3, 0, 2, 512, 8193)
        lens = lens_t.tolist()
        max_ctx, max_pages = 8192, 8192 // jb.PAGE_SIZE
        pool = torch.empty(n * max_pages, 2, Hkv, jb.PAGE_SIZE, D, device="cuda", dtype=torch.bfloat16)
        jb.fill(pool, 3, 1, 0, 0.0, 1.0)
        bt = torch.arange(n * max_pages, dtype=torch.int32, device="cuda").reshape(n, max_pages)
        q = torch.empty(n, Hq * D, device="cuda", dtype=torch.bfloat16); jb.fill(q, 3, 2, 0, 0.0, 1.0)
        ctx = lens_t.cuda()
        out = torch.empty(n, Hq * D, device="cuda", dtype=torch.bfloat16)
        scratch = torch.empty(jb.lib().jsm_attn_decode_scratch_bytes(n, Hq, D, max_ctx) // 4, device="cuda")
        kv_bytes = sum(lens) * Hkv * D * 2 * 2
        cfg = {"workload": "kv_decode_b64_q32_kv8_d128_ctx512-8192", "sum_context": sum(lens), "l2": f"{kv_bytes / 2**20:.0f} MiB of K/V > L2"}
        emit("kv_decode_attention_GBps", timed(lambda _: jb.attn_decode(q, pool, bt, ctx, Hq, Hkv, D, max_ctx, scratch=scratch, out=out)), "hbm", kv_bytes, hbm, "GB/s", cfg)
    return records


def run_timeline(args):
    """Device timeline of the packed projections of one eager decode step (jsm_trace_begin / jsm_trace_end): for every
    projection kind the time its CTAs were resident before their predecessor finished, the main loop, the tail (last
    MMA issued -> last CTA done), and the gap the kernels between two projections leave.  Text output, not a bench line."""
    import numpy as np
    import torch
    import jasmine_b200 as jb
    from jasmine_b200.model import Llama
    torch.cuda.set_device(0)
    B, L = args.batch, min(args.layers, 8)
    tp = max(1, args.tp_emulate)
    m = Llama(L, 4096, 32, 32, 11008, 32000, max_batch=B, max_context=PROMPT + 128, seed=SEED, tp_rank=0, tp_size=tp)
    if tp > 1:
        # one rank of a tensor-parallel group on one GPU: the peers are zero-filled regions of this device whose flags
        # already say "arrived" (no kernel waits for another one); the kernels and their shapes are those of a real
        # rank, the results are not (the peers contribute zeros), the NVLink round trips are absent
        p, nb = C.c_void_p(), C.c_size_t()
        jb.check(jb.lib().jsm_llama_tp_region(m._h, C.byref(p), C.byref(nb)))
        fakes = [torch.zeros(nb.value, dtype=torch.uint8, device="cuda") for _ in range(tp - 1)]
        ptrs = (C.c_void_p * tp)()
        ptrs[0] = p.value
        for r in range(1, tp):
            ptrs[r] = fakes[r - 1].data_ptr()
        flags = torch.full((48,), 1 << 30, dtype=torch.int32)   # the flag words of all exchange protocols: peers "arrived"
        flags[16] = 0                                            # ... but this rank's own push flag is set by its own kernels
        jb.check(jb.lib().jsm_upload(p, flags.data_ptr(), 192, jb.stream_ptr()))
        # exchanges of at most 16 tokens have no flags: their slots hold words {two bf16, epoch}.  The peers' slots of this
        # rank's two push buffers get zeros with a far-future epoch; this rank's own slots stay zero (its own kernels fill them)
        d_model, slot = 4096, 16 * 4096 * 4
        max_tokens = max(B, PROMPT)  # what the model sized its regions for (checked against the region's size)
        assert jb.lib().jsm_tp_region_bytes(max_tokens, d_model) == nb.value, "exchange region: unexpected token capacity"
        words = torch.zeros(slot // 4, dtype=torch.int32)
        words[1::2] = 1 << 30
        words = words.pin_memory()
        for which in range(2):
            for r in range(1, tp):
                off = jb.lib().jsm_tp_inband_slot_offset(which, r, max_tokens, d_model)
                jb.check(jb.lib().jsm_upload(p.value + off, words.data_ptr(), slot, jb.stream_ptr()))
        torch.cuda.synchronize()
        jb.check(jb.lib().jsm_llama_tp_connect(m._h, ptrs))
    nxt = torch.zeros(B, dtype=torch.int32, device="cuda")
    for b in range(B):
        ids = torch.empty(PROMPT, dtype=torch.int32, device="cuda")
        jb.fill(ids, SEED, 5000 + b, 2, 0, 32000)
        m.prefill(ids, b, nxt)
    ids = nxt.clone()
    for _ in range(3):
        m.decode_step(ids, nxt)
        ids.copy_(nxt)
    torch.cuda.synchronize()
    n_max = 4 * L + 1
    jb.check(jb.lib().jsm_trace_begin(n_max))
    m.decode_step(ids, nxt)
    torch.cuda.synchronize()
    buf = np.zeros((n_max, 148, 8), np.uint64)
    n, ctas = C.c_int(), C.c_int()
    jb.check(jb.lib().jsm_trace_end(buf.ctypes.data, n_max, C.byref(n), C.byref(ctas)))
    t = buf[:n.value].astype(np.int64)
    valid = t[:, :, 0] > 0
    names = ["qkv", "wo", "gate/up", "down"]
    mid = range(4, 4 * L - 4)
    print(f"# timeline of one eager decode step, batch {B}, {L} layers of the 7B shape, context {PROMPT + 4}; times in us")
    print("# projection  resident_before_wait  wait->first_stages_landed  wait->last_mma_issued  tail  wait->end  gap_before")
    ends = [t[i][valid[i]][:, 7].max() for i in range(n.value)]
    for k in range(4):
        sel = [i for i in mid if i % 4 == k]
        f = lambda fn: float(np.mean([fn(t[i][valid[i]], i) for i in sel])) / 1e3
        print(f"{names[k]:10s} {f(lambda x, i: x[:, 2].min() - x[:, 0].min()):8.1f} {f(lambda x, i: x[:, 3].max() - x[:, 2].min()):8.1f} "
              f"{f(lambda x, i: x[:, 4].max() - x[:, 2].min()):8.1f} {f(lambda x, i: x[:, 7].max() - x[:, 4].max()):8.1f} "
              f"{f(lambda x, i: x[:, 7].max() - x[:, 2].min()):8.1f} {f(lambda x, i: x[:, 2].min() - ends[i - 1]):8.1f}")
    per_layer = [(ends[4 * (l + 1) + 3] - ends[4 * l + 3]) / 1e3 for l in range(L - 1)]
    print("# per-layer time (us):", " ".join(f"{v:.1f}" for v in per_layer))


# ---- the GPU arm --------------------------------------------------------------------------------------
def tp_parity_check(world, rank, local, dist):
    """TP-N == TP-1 on the GPUs of this run, before anything is timed: a full-width model of a few layers is built as
    the live tensor-parallel group (exchange over peer memory, the product path) and, on rank 0, once more as a single
    rank; both prefill the same prompts (128 tokens: the flash kernel) and run decode steps against the paged cache.
    Returns (on rank 0) the largest logit difference relative to the largest logit, and whether the greedy tokens agree
    wherever the one-rank model's top-2 margin is clear."""
    import torch
    import jasmine_b200 as jb
    from jasmine_b200.model import Llama
    L, B, T, steps = 2, 4, 128, 2
    c = LLAMA7B

    def run(tp_rank, tp_size, connect):
        m = Llama(L, c["d_model"], c["n_heads"], c["n_kv_heads"], c["d_ffn"], c["vocab"], max_batch=B, max_context=T + 16,
                  seed=SEED, tp_rank=tp_rank, tp_size=tp_size)
        if connect:
            m.connect_peers(dist)
        nxt = torch.zeros(B, dtype=torch.int32, device="cuda")
        pre = torch.empty(B, c["vocab"], device="cuda")
        for b in range(B):
            ids = torch.empty(T, dtype=torch.int32, device="cuda")
            jb.fill(ids, SEED, 6000 + b, 2, 0, c["vocab"])
            m.prefill(ids, b, nxt, pre[b])
        out = [pre.clone()]
        lg = torch.empty(B, c["vocab"], device="cuda")
        toks = [nxt.clone()]
        for _ in range(steps):
            ids = nxt.clone()
            m.decode_step(ids, nxt, lg)
            out.append(lg.clone())
            toks.append(nxt.clone())
        # one more step that asks for tokens only: a tensor-parallel group then shares the lm_head by vocabulary and the
        # ranks exchange (best logit, index) pairs; its tokens must be the arg-max of the same step's full logits
        ids = toks[-1].clone()
        tok_only = torch.zeros_like(nxt)
        m.decode_step(ids, tok_only)
        jb.check_device_errors()
        torch.cuda.synchronize()
        out.append(tok_only.clone())
        torch.cuda.synchronize()
        if connect:
            dist.barrier()
        m.close()
        return out, toks

    out_n, tok_n = run(rank, world, True)
    if rank != 0:
        return None
    out_1, tok_1 = run(0, 1, False)
    tok_only_n, tok_only_1 = out_n.pop(), out_1.pop()
    worst, worst_rms, clear_equal, n_clear = 0.0, 0.0, True, 0
    prefix_same = True
    for i, (a, b) in enumerate(zip(out_n, out_1)):
        if not prefix_same:
            break  # the two runs decode different prefixes from here on: nothing to compare
        scale = float(b.abs().max())
        worst = max(worst, float((a - b).abs().max()) / scale)
        worst_rms = max(worst_rms, float((a - b).pow(2).mean().sqrt()) / scale)
        top2 = torch.topk(b, 2, dim=1).values
        clear = (top2[:, 0] - top2[:, 1]) > 2 * 2e-2 * scale
        n_clear += int(clear.sum())
        if bool((tok_n[i][clear] != tok_1[i][clear]).any()):
            clear_equal = False
        prefix_same = bool((tok_n[i] == tok_1[i]).all())
    # the tokens-only step (vocabulary-sharded lm_head + arg-max exchange) against the single rank's tokens of the same step
    sharded_equal = bool((tok_only_n == tok_only_1).all()) if prefix_same else None
    # Both runs are bf16 evaluations of the same function with different summation orders (rank-local products are rounded
    # to bf16 before they are summed); each is held to 2e-2 of the fp32 oracle by the parity tests, so two of them may
    # differ by up to twice that.  The run fails above 4e-2 or on a token mismatch at a clear margin; `within_2e-2` says
    # whether the mutual difference also stays inside the single bar (it does in every run seen: 0.014 - 0.019 at 2, 4 and
    # 8 ranks, which is the rounding noise of the bf16 residual stream, independent of the rank count).
    return {"max_rel_logit_diff": worst, "rms_rel_logit_diff": worst_rms, "within_2e-2": worst <= 2e-2,
            "top1_equal_where_margin_clear": clear_equal, "rows_with_clear_margin": n_clear,
            "sharded_lm_head_tokens_equal": sharded_equal,
            "layers": L, "batch": B, "prompt_len": T, "decode_steps": steps, "tolerance": 4e-2,
            "what": f"logits of a {L}-layer full-width model (d 4096, 32x128 heads, ffn 11008, vocab 32000): the live tp{world} "
                    "group over peer memory against a single rank on rank 0's GPU; prefill + decode steps"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=GEN)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=int(os.environ.get("JSM_BENCH_BATCH", "8")))
    ap.add_argument("--impl", default="jasmine_b200")
    ap.add_argument("--layers", type=int, default=32, help="debug only: fewer layers (the result is then not a bench value)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extras", action="store_true", help="headline only: skip the batch-1/64 legs, the kernel-level legs and the tp parity check")
    ap.add_argument("--workload", default="decode", choices=["decode", "expr", "flash", "kvdecode", "gateup", "timeline"],
                    help="decode = the headline; expr / flash / kvdecode = configurations 2 / 3 / 4 of the baseline "
                         "(kernel-level lines, one JSON line per kernel)")
    ap.add_argument("--tp-emulate", type=int, default=1,
                    help="timeline workload only: run ONE rank of a tensor-parallel group of this size on one GPU")
    ap.add_argument("--profile-steps", type=int, default=0,
                    help="run this many eager decode steps between cudaProfilerStart/Stop and exit (for ncu "
                         "--profile-from-start off); prints no bench line")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    args.warmup = max(args.warmup, 3)
    if args.workload == "timeline":
        return run_timeline(args)
    if args.workload != "decode":
        return run_kernel_workload(args)

    import torch
    import torch.distributed as dist
    import jasmine_b200 as jb
    from jasmine_b200.model import Llama

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        # in-switch (NVLS) reductions bind every rank's buffers to one multicast object; plain peer transfers are used
        # instead so that a rank that leaves abnormally cannot fault the others' GPUs
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    B, K, W = args.batch, args.steps, args.warmup
    extras = not args.no_extras and args.layers == 32 and args.profile_steps == 0
    use_nccl = os.environ.get("JSM_TP_NCCL", "0") == "1"

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    parity = None
    if world > 1 and extras and not use_nccl:
        parity = tp_parity_check(world, rank, local, dist)
        barrier()

    # One model serves every leg: the headline batch, and (extras) batch 1 and batch 64 on the same weights and cache.
    reps = 5 if K < 64 else 1                       # short runs are repeated and the median is reported
    other_batches = [b for b in (1, 64) if b != B] if extras else []
    Ke, Kb = min(K, 64), 32
    max_batch = max([B] + other_batches)
    max_ctx = PROMPT + (W + 2 + reps * K) + (Ke + 2) + len(other_batches) * (W + 2 + Kb) + 24
    cfg = dict(LLAMA7B, n_layers=args.layers)
    model = Llama(cfg["n_layers"], cfg["d_model"], cfg["n_heads"], cfg["n_kv_heads"], cfg["d_ffn"], cfg["vocab"],
                  max_batch=max_batch, max_context=max_ctx, seed=SEED, tp_rank=rank, tp_size=world)
    if world > 1:
        def allreduce(ptr, count, dtype, stream):
            iface = {"shape": (count,), "typestr": "<u2" if dtype == jb.BF16 else "<f4", "data": (ptr, False), "version": 2}
            holder = type("DevBuf", (), {"__cuda_array_interface__": iface})()
            t = torch.as_tensor(holder, device="cuda")
            if dtype == jb.BF16:
                t = t.view(torch.bfloat16)
            dist.all_reduce(t)
        model.set_allreduce(allreduce)
        if not use_nccl:
            # the product path: the model's own exchange over peer memory (NCCL stays as the plumbing and, with
            # JSM_TP_NCCL=1, as the comparison)
            model.connect_peers(dist)

    # synthetic prompts: max_batch sequences of PROMPT token ids, uniform in [0, vocab)
    nxt = torch.zeros(max_batch, dtype=torch.int32, device="cuda")
    t_pre0 = time.perf_counter()
    for b in range(max_batch):
        ids = torch.empty(PROMPT, dtype=torch.int32, device="cuda")
        jb.fill(ids, SEED, 5000 + b, 2, 0, cfg["vocab"])
        model.prefill(ids, b, nxt)
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t_pre0
    ids = nxt.clone()
    ctx = [PROMPT] * max_batch                      # host copy of the context lengths (the device keeps its own)

    def timed_decode(Bt, Kt, Wt, n_reps, sample_clocks):
        """Wt eager warm-up steps, then n_reps times Kt replays of the captured step of batch Bt; device time (CUDA events,
        max over ranks) of the median repetition, the mean context length of that repetition, launches per step."""
        ids_b, nxt_b = ids[:Bt], nxt[:Bt]
        launches0 = jb.launch_count()
        for i in range(Wt):
            model.decode_step(ids_b, nxt_b)
            ids_b.copy_(nxt_b)
            if i == 0:
                jb.check_device_errors()  # a bounded device-side wait that ran out (a peer that never arrived) stops the run here
        torch.cuda.synchronize()
        per_step = (jb.launch_count() - launches0) // Wt
        graph = None
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    model.decode_step(ids_b, nxt_b)
                    ids_b.copy_(nxt_b)
            torch.cuda.current_stream().wait_stream(side)
            graph = g
        except Exception as e:  # multi-rank capture of the collective can be refused: run the step eagerly
            if rank == 0:
                print(f"# graph capture failed ({type(e).__name__}: {e}); timing eager steps", file=sys.stderr)
            torch.cuda.synchronize()

        def one_step():
            if graph is not None:
                graph.replay()
            else:
                model.decode_step(ids_b, nxt_b)
                ids_b.copy_(nxt_b)
        one_step()  # one replay outside the timed region
        for b in range(Bt):
            ctx[b] += Wt + 1
        clocks = ClockSampler(local) if sample_clocks else None
        barrier()
        if clocks is not None and rank == 0:
            clocks.start()
        runs = []
        for _ in range(n_reps):
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            ev0.record()
            for _ in range(Kt):
                one_step()
            ev1.record()
            barrier()
            runs.append((max_over_ranks(ev0.elapsed_time(ev1)), sum(ctx[:Bt]) / Bt + (Kt + 1) / 2.0))
            for b in range(Bt):
                ctx[b] += Kt
        clock_info = clocks.stop() if (clocks is not None and rank == 0) else None
        jb.check_device_errors()
        runs_sorted = sorted(runs)
        ms, ctx_mid = runs_sorted[len(runs_sorted) // 2]
        return {"ms": ms, "ctx_mid": ctx_mid, "launches_per_step": per_step, "graph": graph, "clocks": clock_info,
                "all_ms_per_step": [r[0] / Kt for r in runs]}

    if args.profile_steps > 0:
        for _ in range(W):
            model.decode_step(ids[:B], nxt[:B])
            ids[:B].copy_(nxt[:B])
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        for _ in range(args.profile_steps):
            model.decode_step(ids[:B], nxt[:B])
            ids[:B].copy_(nxt[:B])
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(f"# profiled {args.profile_steps} eager decode steps", file=sys.stderr)
        return

    peak, peak_kind = measured_peaks()
    wbytes, kv_per_tok = model.step_bytes()

    def step_roofline(Bt, ms_per_step, ctx_mid):
        nbytes = wbytes + Bt * ctx_mid * kv_per_tok
        gbs = nbytes / (ms_per_step * 1e-3) / 1e9
        return {"bytes_per_step": nbytes, "achieved_gbs": gbs, "frac": gbs / peak}

    head = timed_decode(B, K, W, reps, True)
    ms = head["ms"]
    graph = head["graph"]
    tok_s = B * K / (ms / 1e3)
    last_tokens = nxt[:min(B, 8)].tolist()

    # end to end through the C ABI with HOST buffers: jsm_llama_decode_step_host takes the ids from (pinned) host memory,
    # replays the graph the library captured for this batch size and hands the next tokens back to host memory, every step
    h_ids = torch.empty(B, dtype=torch.int32).pin_memory()
    h_next = torch.empty(B, dtype=torch.int32).pin_memory()
    h_ids.copy_(ids[:B].cpu())
    # the same steps as the reported (median) repetition: the context lengths go back to where that repetition began
    # (jsm_llama_set_context; the cache entries from there on are written again), and forward again afterwards
    torch.cuda.synchronize()
    ctx_end = list(ctx[:B])
    for b in range(B):
        ctx[b] = ctx_end[b] - (reps - reps // 2) * K + (K - Ke) // 2   # (centred when the leg is shorter than the repetition)
        model.set_context(b, ctx[b])
    e2e_stream = torch.cuda.Stream()
    with torch.cuda.stream(e2e_stream):
        for _ in range(2):  # the first call captures
            model.decode_step_host(h_ids, h_next)
            h_ids.copy_(h_next)
        barrier()
        t0 = time.perf_counter()
        for _ in range(Ke):
            model.decode_step_host(h_ids, h_next)
            h_ids.copy_(h_next)
        e2e_s = time.perf_counter() - t0
    barrier()
    torch.cuda.synchronize()
    for b in range(B):
        ctx[b] = max(ctx[b] + Ke + 2, ctx_end[b])
        model.set_context(b, ctx[b])
    e2e_s = max_over_ranks(e2e_s)
    e2e_tok_s = B * Ke / e2e_s
    ids[:B].copy_(h_ids)

    batches = {}
    for ob in other_batches:
        r = timed_decode(ob, Kb, W, 1, False)
        r.pop("graph")
        ms_b = r["ms"] / Kb
        batches[str(ob)] = {"tok_s": ob * Kb / (r["ms"] / 1e3), "ms_per_step": ms_b, "steps": Kb,
                            "launches_per_step": r["launches_per_step"], "mean_context": r["ctx_mid"],
                            "step_roofline": step_roofline(ob, ms_b, r["ctx_mid"])}

    if rank != 0:
        shutdown(graph)
        return

    # roofline of the dominant kernel, timed alone: the SwiGLU gate/up weight stream of one layer
    # (2 x 11008 x 4096 bf16 = 180 MB per launch over packed weights, 4 rotating weight sets: larger than L2)
    d, ffn_l = cfg["d_model"], cfg["d_ffn"] // world
    x = torch.empty(B, d, device="cuda", dtype=torch.bfloat16)
    jb.fill(x, SEED, 7000, 0, 0.0, 1.0)
    y = torch.empty(B, ffn_l, device="cuda", dtype=torch.bfloat16)
    packed_sets = []
    for i in range(4):
        w = torch.empty(2 * ffn_l, d, device="cuda", dtype=torch.bfloat16)
        jb.fill(w, SEED, 9000 + i, 0, 0.0, 0.02)
        packed_sets.append(jb.linear_pack(w, ffn_l, paired=True))
        del w

    def stream_once(i, fn):
        jb.check(fn(x.data_ptr(), packed_sets[i].data_ptr(), None, 3, None, y.data_ptr(), jb.BF16, B, ffn_l, d, jb.stream_ptr()))

    def time_launches(fn, n_launch=96):
        for i in range(4):
            stream_once(i, fn)
        torch.cuda.synchronize()
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        r0.record()
        for i in range(n_launch):
            stream_once(i % 4, fn)
        r1.record()
        torch.cuda.synchronize()
        return r0.elapsed_time(r1) / n_launch

    # launched the way the decode step launches it (jsm_linear_bf16_packed_chained: every launch a link of a kernel chain,
    # resident and requesting its first weights while its predecessor finishes), and as plain stream-ordered launches
    k_ms = time_launches(jb.lib().jsm_linear_bf16_packed_chained)
    k_ms_plain = time_launches(jb.lib().jsm_linear_bf16_packed)
    alg_bytes = 2 * ffn_l * d * 2 + B * d * 2 + B * ffn_l * 2
    achieved = alg_bytes / (k_ms * 1e-3) / 1e9
    achieved_plain = alg_bytes / (k_ms_plain * 1e-3) / 1e9
    # the same kernel inside the step (chained launches: its ring is full of weights when its predecessor ends): device
    # time stamps of one eager step, predecessor end -> last CTA done, mean over the gate/up launches of the layers
    in_step = None
    if world == 1 and cfg["n_layers"] >= 4:
        import numpy as np
        n_max = 4 * cfg["n_layers"] + 1
        jb.check(jb.lib().jsm_trace_begin(n_max))
        model.decode_step(ids[:B], nxt[:B])
        torch.cuda.synchronize()
        buf = np.zeros((n_max, 148, 8), np.uint64)
        n_tr, n_ctas = C.c_int(), C.c_int()
        jb.check(jb.lib().jsm_trace_end(buf.ctypes.data, n_max, C.byref(n_tr), C.byref(n_ctas)))
        tr = buf[:n_tr.value].astype(np.int64)
        spans = []
        for i in range(6, n_tr.value - 1, 4):  # launch 4l+2 of layer l is the gate/up projection
            v = tr[i][tr[i][:, 0] > 0]
            if len(v):
                spans.append((v[:, 7].max() - v[:, 2].min()) / 1e6)
        if spans:
            ms_in = float(np.mean(spans))
            in_step = {"ms_per_launch": ms_in, "achieved": alg_bytes / (ms_in * 1e-3) / 1e9,
                       "how": "device time stamps (globaltimer) of one eager decode step: predecessor kernel finished -> last "
                              "CTA of the gate/up projection done, mean over the layers"}
            in_step["frac"] = in_step["achieved"] / peak
    del packed_sets

    # DRAM traffic of one launch of this kernel from an ncu capture (dram__bytes_read.sum + dram__bytes_write.sum): the
    # capture is of the 8-token, one-GPU shape only; any other run reports none
    traffic = 184.7e6 if (world == 1 and B == 8) else None
    line = {
        "metric": "llama7b_decode_tokens_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(args, world),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic,
                     "traffic_note": "measured under ncu for one launch of this kernel at 8 tokens on one GPU; null for any other shape",
                     "kernel": "linear_packed_kernel: gate/up projection weight stream (jsm_linear_bf16_packed, silu*up epilogue)",
                     "peak_source": f"{peak_kind} HBM copy bandwidth", "ms_per_launch": k_ms, "bytes_per_launch": alg_bytes,
                     "timed": "this kernel alone, CUDA events around 96 back-to-back launches over 4 rotating weight sets, launched as "
                              "the decode step launches it (jsm_linear_bf16_packed_chained: programmatic dependent launch, a launch "
                              "sets up and requests its first weights during its predecessor's tail); elapsed / launches",
                     "plain_launches": {"ms_per_launch": k_ms_plain, "achieved": achieved_plain, "frac": achieved_plain / peak,
                                        "how": "the same 96 launches through jsm_linear_bf16_packed (plain stream order: each "
                                               "launch starts after its predecessor has ended)"},
                     "in_step": in_step},
        "step_roofline": dict(step_roofline(B, ms / K, head["ctx_mid"]),
                              note="all streamed weights (every projection and lm_head) + cached K/V of the step over the measured step time"),
        "repetitions": {"n": reps, "ms_per_step": head["all_ms_per_step"], "reported": "median"},
        "e2e": {"value": e2e_tok_s, "unit": "tok/s", "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B, "steps": Ke,
                "how": "jsm_llama_decode_step_host: ids from pinned host memory, library-owned CUDA graph of the step, next tokens "
                       "back to host memory and a stream synchronisation, every step; over the same context lengths as the "
                       "reported repetition of `value`"},
        "gpu_launches": head["launches_per_step"] * K, "launches_per_step": head["launches_per_step"], "cuda_graph": graph is not None,
        "prefill_s": prefill_s, "clocks": head["clocks"],
        # greedy tokens of the last timed step (first 8 sequences).  Random-init logits are nearly flat, so after dozens of
        # steps these differ between GPU counts through bf16 summation order alone: they identify a run, they prove no
        # parity.  Parity across GPU counts is what `tp_parity` measures.
        "last_tokens": last_tokens,
    }
    if batches:
        line["batches"] = batches
    if parity is not None:
        line["tp_parity"] = parity
    if args.layers != 32:
        line["invalid"] = "debug run with fewer layers"
    if extras and world == 1:
        # configurations 2, 3 and 4 of the baseline as kernel-level legs (a few seconds): the model's memory is released first
        shutdown_model = model
        del graph
        head["graph"] = None
        shutdown_model.close()
        torch.cuda.empty_cache()
        kernels = {}
        for wl in ("expr", "flash", "kvdecode"):
            sub = argparse.Namespace(**vars(args))
            sub.workload, sub.steps, sub.warmup = wl, 20, 3
            try:
                for rec in run_kernel_workload(sub, collect=True):
                    kernels[rec["metric"]] = {"value": rec["value"], "unit": rec["unit"], "ms": rec["ms_per_step"],
                                              "frac_of_peak": rec["roofline"]["frac"], "peak": rec["roofline"]["peak"],
                                              "workload": rec["config"]["workload"]}
            except Exception as e:
                kernels[wl] = {"failed": f"{type(e).__name__}: {e}"}
        line["kernels"] = kernels
        graph = None
    if not args.no_cpu and world == 1:
        try:
            line["cpu_baseline"] = cpu_port_baseline()
        except Exception as e:
            line["cpu_baseline"] = {"value": None, "unit": "tok/s", "cores": os.cpu_count(), "kind": "port",
                                    "sample": f"failed: {type(e).__name__}: {e}"}
    bad_parity = parity is not None and (parity["max_rel_logit_diff"] > parity["tolerance"] or not parity["top1_equal_where_margin_clear"]
                                         or parity["sharded_lm_head_tokens_equal"] is False)
    if bad_parity:
        line["invalid"] = "tensor-parallel parity check failed"
    print(json.dumps(line), flush=True)
    shutdown(graph)
    if bad_parity:
        sys.exit(3)


def shutdown(graph):
    """Leaves a multi-rank run without waiting on the communicator: tearing down a process group whose collectives
    live in a captured graph has blocked forever here, so the graph is dropped first and the process then exits
    by the regular tear-down; if that still blocks, the process exits after 20 s (all ranks are past their last
    collective and a final barrier by then)."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return
    del graph
    torch.cuda.synchronize()
    dist.barrier()  # every rank has finished its work: nobody leaves while another still computes
    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()

    def give_up():
        time.sleep(20.0)
        os._exit(0)
    threading.Thread(target=give_up, daemon=True).start()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
