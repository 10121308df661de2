#!/usr/bin/env python
"""Benchmark of the B200 ternary decode path.

Workload "falcon3_10b_gemv_sweep": the 280 ternary projections of one Falcon3-10B decode step at batch 1 (40 layers x
q, k, v, o, gate, up, down), each with its own seeded int8 activation vector, weights resident in HBM (1.9 GB, far
beyond L2). One step = one pass over all 280 projections = the velurex bytes of one decoded token.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

Prints ONE JSON line (rank 0). With --impl reference the CPU restatement of the reference's AVX-512 kernel is timed on
the host cores instead (the reference itself is Rust and cannot be built here).
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

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from quintrit_b200 import synth  # noqa: E402

CONFIG_ID = 0
BYTES_PER_WEIGHT = 0.2  # 1.60 bits per weight: the algorithmic bytes of a velurex GEMV
# DRAM bytes per weight that ncu counted for gemv_lut_kernel (dram__bytes_read.sum + dram__bytes_write.sum of a capture of
# the 12-layer case, divided by its 2 850 029 568 weights); traffic grows in proportion to the weights streamed, so a
# launch's traffic is this figure times its weights.
NCU_TRAFFIC_BYTES_PER_WEIGHT = (590_314_496 + 4_031_488) / 2_850_029_568


def sweep_shapes(layers: int):
    return [(l, p, n, k) for l in range(layers) for p, (n, k) in enumerate(synth.falcon3_10b_shapes())]


def shard_rows(n: int, rank: int, world: int):
    """Rows [r0, r1) of a projection that rank `rank` of `world` streams: whole 32-row tiles, remainder to the low ranks."""
    tiles = -(-n // 32)
    t0 = tiles * rank // world
    t1 = tiles * (rank + 1) // world
    return min(t0 * 32, n), min(t1 * 32, n)


def shard_plan(layers: int, rank: int, world: int):
    """What rank `rank` of `world` streams, as (layer, projection, first row, end row, columns) per work unit, and the name of the rule.

    The projections of the sweep are independent objects. When the layers divide evenly, a rank takes whole layers (every layer has the same
    weights, so the shares are equal and every matrix keeps its full height: the kernel builds one activation table per pair of 160-column blocks
    and reuses it for all rows it streams, so short matrices cost more per weight); otherwise every projection is cut by rows. Neither
    needs a collective."""
    shapes = sweep_shapes(layers)
    if world > 1 and layers % world == 0:
        per = layers // world
        return [(l, p, 0, n, k) for (l, p, n, k) in shapes if rank * per <= l < (rank + 1) * per], f"layers/{world}"
    out = []
    for (l, p, n, k) in shapes:
        r0, r1 = shard_rows(n, rank, world)
        if r1 > r0:
            out.append((l, p, r0, r1, k))
    return out, f"rows/{world}"


def activations_for(layer: int, proj: int, cols: int) -> np.ndarray:
    x = synth.normal_f32(synth.seed_for(CONFIG_ID, layer, proj, 2), cols)
    return synth.quantize_int8_np(x)[0]


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons in the background. Samples are kept if their timestamp falls
    inside the load window [mark_begin, mark_end] that the caller brackets around the timed region."""

    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None
        self.t0 = self.t1 = None

    def start(self, wait_s: float = 5.0):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self.gpu_index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
            t = time.time()
            while time.time() - t < wait_s and os.path.getsize(self.path) == 0:
                time.sleep(0.05)
        except Exception:
            self.proc = None

    def mark_begin(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def stop(self):
        import datetime

        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    if self.t0 is not None and not (self.t0 <= ts <= (self.t1 or ts) + 0.05):
                        continue
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                    pw.append(float(f[3]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm), power_w_max=max(pw))
        return out


class CpuSweep:
    """The sweep on the host cores: the CPU restatement of the reference's AVX-512 kernel (oracle/cpu_gemv.c) over the first
    `layers` layers of the sweep in the 64-row tile layout. The weights come from the oracle library's threaded generator
    (the same seeded stream as the GPU arm's)."""

    def __init__(self, layers: int):
        import oracle

        self.oracle = oracle
        self.use512 = oracle.cpu_has_avx512_vbmi()
        self.probs = []
        for (l, p, n, k) in sweep_shapes(layers):
            planar = oracle.synth_planar(synth.seed_for(CONFIG_ID, l, p, 0), n, k)
            w = oracle.tile64(planar, n, k) if self.use512 else planar
            self.probs.append((n, k, w, activations_for(l, p, k), np.zeros(n, np.int32)))
        self.weights = sum(n * k for n, k, *_ in self.probs)
        self.fn = oracle.cpu_gemv_avx512 if self.use512 else oracle.cpu_gemv_portable
        self.isa = "avx512_vbmi" if self.use512 else "portable"

    def one_pass(self, threads: int, reverse: bool = False) -> float:
        order = range(len(self.probs) - 1, -1, -1) if reverse else range(len(self.probs))
        t0 = time.perf_counter()
        for i in order:
            n, k, w, a, o = self.probs[i]
            self.fn(w, n, k, a, threads, out=o)
        return time.perf_counter() - t0

    def best_of(self, threads: int, reps: int = 9) -> float:
        """Gweights/s by the reference's method (docs/benchmarks.md:45-59): best of `reps` passes, averaged over two rounds
        with the second in reverse order."""
        self.one_pass(threads)
        best1 = min(self.one_pass(threads) for _ in range(reps))
        best2 = min(self.one_pass(threads, reverse=True) for _ in range(reps))
        return self.weights / (0.5 * (best1 + best2)) / 1e9

    def results(self):
        return [p[4] for p in self.probs]


def pin_to_all_cores():
    """Keeps the process (and the OpenMP threads it starts) on the cores it may use, one thread per core, no migration
    (the reference pins its pool with QUINTRIT_POOL_PIN=1). Must run before the oracle library is first used."""
    os.environ.setdefault("OMP_PROC_BIND", "close")
    os.environ.setdefault("OMP_PLACES", "cores")
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def sweep_config(layers: int, world: int, weights_total: int) -> dict:
    """The `config` object of the sweep line; both arms print the same one."""
    return {"workload": "falcon3_10b_gemv_sweep", "layers": layers, "projections": 7 * layers, "batch": 1, "weights": weights_total,
            "l2": f"inputs ({weights_total * BYTES_PER_WEIGHT / 1e9:.1f} GB of weights per pass over all GPUs) exceed L2", "sharding": f"{shard_plan(layers, 0, world)[1]}, no collective"}


def run_decode(args, local_rank: int):
    """Whole-token decode of the Falcon3-10B shape (or --decode-shape) at batch 1 on one GPU: device time per token at a
    context of --prompt tokens, end-to-end time per token through the C ABI, and a greedy-token parity check."""
    import torch

    import quintrit_b200 as q

    dev = torch.device("cuda", local_rank)
    ctx = (max(args.prompt + args.steps + 64, args.parity_prompt + args.parity_new + 1) + 255) // 256 * 256
    if args.batch_seqs > 0:  # the sequences of the batched leg: prompts of 256 .. 2048 tokens and the generated tokens behind them
        ctx = max(ctx, (2048 + args.batch_steps + 8 + 255) // 256 * 256)
    t0 = time.time()
    spec = synth.torch_model(args.decode_shape, dev, ctx, layers=args.decode_layers)
    torch.cuda.empty_cache()
    dec = q.Decoder(spec, device=local_rank)
    setup_s = time.time() - t0
    weights = sum(int(np.prod(sh)) for sh in [(spec["q_heads"] * spec["head_dim"], spec["hidden"]), (spec["kv_heads"] * spec["head_dim"], spec["hidden"]),
                                               (spec["kv_heads"] * spec["head_dim"], spec["hidden"]), (spec["hidden"], spec["q_heads"] * spec["head_dim"]),
                                               (spec["inter"], spec["hidden"]), (spec["inter"], spec["hidden"]), (spec["hidden"], spec["inter"])]) * spec["layers"]
    if args.batch_only:  # profiling aid: the batched-decode leg alone
        out = {"shape": spec["shape"], "layers": spec["layers"], "batched_decode": run_batched_decode(args, dec, spec, None)}
        dec.free()
        return out
    prompt = synth.prompt_tokens(2, args.prompt, spec["vocab"])
    # parity leg: a short prompt and a few greedy tokens against the CPU oracle (same arrays)
    parity = None
    if not args.no_cpu:
        import oracle

        ref = oracle.Model(spec)
        npar, ngen = args.parity_prompt, args.parity_new  # the full-length sequences are checked against committed fixtures by --parity-full
        tok = None
        t_cpu = time.time()
        for pos in range(npar):
            tok = oracle.argmax(ref.forward(int(prompt[pos]), pos))
        want = [tok]
        for j in range(1, ngen):
            tok = oracle.argmax(ref.forward(int(tok), npar + j - 1))
            want.append(tok)
        cpu_tok_s = (npar + ngen - 1) / (time.time() - t_cpu)
        got = dec.generate(prompt[:npar], ngen)
        lg_ref = ref.forward(int(got[-1]), npar + ngen - 1)
        lg_gpu, _ = dec.forward(int(got[-1]), npar + ngen - 1)
        parity = {"greedy_tokens_checked": ngen, "identical": bool(list(got) == want), "logits_bit_exact": bool(np.array_equal(lg_ref.view(np.uint32), lg_gpu.view(np.uint32))),
                  "cpu_tokens_per_s": round(cpu_tok_s, 2), "cpu_threads": os.cpu_count()}
        del ref
    # ingest the prompt: token by token on the device (the reference's way), and in chunks on the tensor cores; both must end in the same token
    t0 = time.perf_counter()
    first = dec.generate(prompt, 1)
    serial_s = time.perf_counter() - t0
    ingest = None
    try:
        dec.prefill(prompt[:16])  # makes the two-bit copies of the weights and the chunk buffers
        t0 = time.perf_counter()
        _, nxt = dec.prefill(prompt)  # the first prompt: its second full chunk is captured into the graph that later chunks replay
        first_s = time.perf_counter() - t0
        t0 = time.perf_counter()
        _, nxt2 = dec.prefill(prompt)
        chunk_s = time.perf_counter() - t0
        ingest = {"prompt_tokens": int(len(prompt)), "token_by_token_tokens_per_s": round(len(prompt) / serial_s, 1), "chunked_tokens_per_s": round(len(prompt) / chunk_s, 1),
                  "chunked_ms": round(chunk_s * 1e3, 2), "first_prompt_ms": round(first_s * 1e3, 2), "chunk": 256, "same_next_token": bool(int(nxt) == int(first[0]) == int(nxt2)),
                  "kernel": "gemm_i8_tcgen05_kernel for the projections, the step kernels with a token index in the grid"}
    except q.QuintritError as e:
        ingest = {"error": str(e)}
    q.launch_count(reset=True)
    dec.time_token(1, max(3, args.warmup))
    launches_per_token = q.launch_count() / max(3, args.warmup)
    step_ms = dec.time_token(1, args.steps)          # exactly K steps, CUDA events on the decoder's stream
    best_ms = dec.time_token(5, max(args.steps, 50))  # the reference's method: minimum over blocks of replays
    # end to end: token id in from the host, greedy token out to the host, every step
    tok, pos = int(first[0]), args.prompt
    t1 = time.perf_counter()
    for _ in range(args.steps):
        _, tok = dec.forward(tok, pos, want_logits=False)
        pos += 1
    e2e_ms = (time.perf_counter() - t1) * 1e3 / args.steps
    bytes_tok = weights * BYTES_PER_WEIGHT
    out = {
        "shape": spec["shape"], "layers": spec["layers"], "context": args.prompt, "tokens_per_s": round(1e3 / step_ms, 1), "ms_per_token": round(step_ms, 4),
        "best_ms_per_token": round(best_ms, 4), "velurex_bytes_per_token": int(bytes_tok),
        "roofline_nominal_8tbs_frac": round(bytes_tok / (step_ms * 1e-3) / 8e12, 4),
        "hbm_frac_of_measured": round(bytes_tok / (step_ms * 1e-3) / 1e9 / measured_peaks()[0], 4),
        "e2e": {"tokens_per_s": round(1e3 / e2e_ms, 1), "ms_per_token": round(e2e_ms, 4), "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 8},
        "kernel_launches_per_token": round(launches_per_token, 1), "setup_s": round(setup_s, 1), "parity_vs_cpu": parity, "prompt_ingestion": ingest,
    }
    if args.batch_seqs > 0:
        try:
            out["batched_decode"] = run_batched_decode(args, dec, spec, step_ms)
        except q.QuintritError as e:
            out["batched_decode"] = {"error": str(e)}
    dec.free()
    return out


def run_batched_decode(args, dec, spec, single_ms: float):
    """Several sequences with prompts of different lengths decoded together (one batched pass over the weights per step): aggregate tokens/s of
    the greedy steps, wall clock around the C call with the chosen tokens read back every step, and a check of two sequences against the
    same sequences decoded alone."""
    import torch

    import quintrit_b200 as q

    n_seq, steps = args.batch_seqs, args.batch_steps
    lengths = synth.batch_lengths(3, n_seq)
    prompts = [synth.prompt_tokens(100 + i, int(n), spec["vocab"]) for i, n in enumerate(lengths)]
    batch = q.Batch(dec, n_seq)
    t0 = time.perf_counter()
    first = [batch.prefill(i, p)[1] for i, p in enumerate(prompts)]
    ingest_s = time.perf_counter() - t0
    check = sorted(range(n_seq), key=lambda i: lengths[i])[:2]  # the two shortest: decoded alone afterwards, token by token
    for _ in range(3):
        batch.step()
    got = {i: [] for i in check}
    torch.cuda.profiler.start()  # a profiler started with "--profile-from-start off" sees the timed steps only; a no-op otherwise
    t0 = time.perf_counter()
    for k in range(steps):
        toks, _ = batch.step()
        for i in check:
            got[i].append(int(toks[i]))
    step_s = (time.perf_counter() - t0) / steps
    torch.cuda.profiler.stop()
    batch.free()
    same = True
    for i in check:
        _, tok = dec.prefill(prompts[i])
        same = same and int(tok) == int(first[i])
        alone = []
        for k in range(3 + steps):
            _, tok = dec.forward(int(tok), int(lengths[i]) + k, want_logits=False)
            alone.append(int(tok))
        same = same and alone[3:] == got[i]
    return {"sequences": n_seq, "prompt_lengths": "uniform in [256, 2048] (stream 4)", "prompt_tokens_total": int(lengths.sum()), "mean_context": round(float(lengths.mean()), 1),
            "steps": steps, "ms_per_step": round(step_s * 1e3, 3), "tokens_per_s": round(n_seq / step_s, 1), "speedup_vs_one_sequence": None if single_ms is None else round(n_seq / step_s / (1e3 / single_ms), 2),
            "prompt_ingestion_tokens_per_s": round(float(lengths.sum()) / ingest_s, 1), "sequences_checked_against_decoding_alone": len(check), "identical_tokens": bool(same),
            "timing": "wall clock around quintrit_b200_batch_step, the chosen tokens copied to the host every step"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def run_decode_tp(args, rank: int, world: int, local_rank: int, dist):
    """Whole-token decode of the Falcon3-10B shape split over `world` GPUs (tensor parallel: every rank streams 1/world of
    every projection; slices are exchanged inside the token kernel over NVLink peer stores). Every rank calls this; rank 0
    returns the result object. Parity: the group's greedy tokens against a one-GPU decoder of the whole model on rank 0."""
    import torch

    import quintrit_b200 as q

    dev = torch.device("cuda", local_rank)
    ctx = (args.prompt + args.steps + 64 + 255) // 256 * 256
    shape = {"falcon3_10b": (12, 4, 3072, 23040, 131072), "bitnet_2b": (20, 5, 2560, 6912, 128256)}[args.decode_shape]
    if args.decode_shape != "falcon3_10b" or shape[2] % world or shape[3] % world or shape[4] % world:
        return {"tp_world": world, "skipped": f"tensor-parallel decode is built for the LLaMA / Falcon3 architecture with {world} dividing hidden, FFN and vocabulary sizes"} if rank == 0 else None
    npar, ngen = 6, 6
    short = synth.prompt_tokens(2, npar, shape[4])
    want = None
    if rank == 0:  # the one-GPU answer for the same seeded model
        full = synth.torch_model(args.decode_shape, dev, ctx, layers=args.decode_layers)
        one = q.Decoder(full, device=local_rank)
        want = [int(t) for t in one.generate(short, ngen)]
        one.free()
        del full, one
        torch.cuda.empty_cache()
    dist.barrier()
    t0 = time.time()
    spec = synth.torch_model(args.decode_shape, dev, ctx, layers=args.decode_layers, tp=(rank, world))
    dec = q.Decoder(spec, device=local_rank)
    handles = [None] * world
    dist.all_gather_object(handles, dec.tp_handle())
    dec.tp_attach(handles)
    dist.barrier()  # every rank has mapped every box before the first token kernel starts
    setup_s = time.time() - t0
    got = [int(t) for t in dec.generate(short, ngen)]
    gathered = [None] * world
    dist.all_gather_object(gathered, got)
    prompt = synth.prompt_tokens(2, args.prompt, spec["vocab"])
    dec.generate(prompt, 1)
    dist.barrier()
    dec.time_token(1, max(3, args.warmup))
    dist.barrier()
    step_ms = dec.time_token(1, args.steps)
    best_ms = dec.time_token(5, max(args.steps, 50))
    t = torch.tensor([step_ms, best_ms], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    step_ms, best_ms = t.tolist()
    dist.barrier()
    dec.free()
    if rank != 0:
        return None
    weights = sum(n * k for _, _, n, k in sweep_shapes(spec["layers"]))
    bytes_tok = weights * BYTES_PER_WEIGHT
    return {"shape": spec["shape"], "layers": spec["layers"], "context": args.prompt, "tp_world": world, "tokens_per_s": round(1e3 / step_ms, 1),
            "ms_per_token": round(step_ms, 4), "best_ms_per_token": round(best_ms, 4), "velurex_bytes_per_token": int(bytes_tok),
            "roofline_nominal_8tbs_frac": round(bytes_tok / (step_ms * 1e-3) / (world * 8e12), 4), "exchanges_per_token": (3 if shape[1] % world else 4) * spec["layers"] + 1, "attention": "replicated on every rank (the ranks do not divide the KV heads)" if shape[1] % world else "split by KV head",
            "transport": "8-byte (value, sequence) peer stores into every rank's box inside the token kernel, polled by the readers",
            "parity": {"greedy_tokens_checked": ngen, "all_ranks_agree": all(g == got for g in gathered), "identical_to_one_gpu": got == want},
            "setup_s": round(setup_s, 1)}


def run_block_scaled(args, local_rank: int):
    """The block-scaled (Q2_0 x Q8_0) projection on the three Falcon3-10B projection shapes through the C ABI with host
    buffers (activations in, results out, every call). Profiling aid: the kernel's device time is read from an ncu launch
    list of this command."""
    import quintrit_b200 as q
    from quintrit_b200 import gguf_io

    out = []
    for rows, cols in [(3072, 3072), (23040, 3072), (3072, 23040)]:
        rng = np.random.default_rng(rows + cols)
        trits = rng.integers(-1, 2, size=(rows, cols)).astype(np.int8)
        sc = rng.uniform(0.5, 2.0, rows * cols // 64).astype(np.float16)
        m = q.Matrix(gguf_io.encode_q2_0(trits, sc), rows, cols, q.SRC_Q2_0, device=local_rank)
        x = rng.standard_normal(cols).astype(np.float32)
        for _ in range(max(3, args.warmup)):
            m.gemv_block_scaled(x)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            m.gemv_block_scaled(x)
        dt = (time.perf_counter() - t0) / args.steps
        out.append({"rows": rows, "cols": cols, "us_per_call_host_buffers": round(dt * 1e6, 1), "gweights_per_s": round(rows * cols / dt / 1e9, 1)})
        m.free()
    return out


def run_block_scaled_decode(args, local_rank: int):
    """Whole-token decode of a block-scaled (Q2_0) model of the decode shape, loaded from a synthetic GGUF file, at context
    --prompt; --decode-layers layers (default 4: a launch list needs no more). The two steps between the profiler marks are the
    ones an ncu launch list with --profile-from-start off sees; the time is read with the decoder's own device timer."""
    import tempfile

    import torch

    import quintrit_b200 as q
    from quintrit_b200 import gguf_io, synth

    layers = args.decode_layers or 4
    ctx = (args.prompt + 256) // 256 * 256
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "m.gguf")
        d = gguf_io.write_full_model_gguf(path, args.decode_shape, gguf_io.GGML_Q2_0, torch.device("cuda", local_rank), ctx, layers=layers)
        torch.cuda.empty_cache()
        dec = q.Decoder.open(path, context=ctx, device=local_rank)
    got = dec.generate(synth.prompt_tokens(d["config"], args.prompt - 1, d["vocab"]), 1)
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    for i in range(2):
        dec.forward(int(got[-1]), args.prompt - 1 + i, want_logits=False)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    ms = dec.time_token(3, 20)
    out = {"model": args.decode_shape, "encoding": "q2_0", "layers": layers, "context": args.prompt + 1, "ms_per_token": round(ms, 4),
           "single_kernel": dec.info()["single_kernel"]}
    dec.free()
    return out


def run_moe(args, local_rank: int):
    """One mixture-of-experts feed-forward block of the Qwen3-30B-A3B shape (hidden 2048, 128 experts of width 768, top-8 softmax routing,
    BF16 router, ternary experts) for a batch of 16 tokens on one GPU: device time of the block's launches, the time of the C call with host
    buffers, and two tokens checked against the composition of the reference's pieces (oracle/moe.py). The block only: attention, norms and
    the exchange between GPUs of an expert-parallel model are not part of it."""
    import torch

    import quintrit_b200 as q

    dev = torch.device("cuda", local_rank)
    H, I, E, K, B = 2048, 768, 128, 8, 16
    cfg = 4
    t0 = time.time()
    gu, dn, scales = [], [], []
    for e in range(E):
        g = synth.torch_planar(synth.seed_for(cfg, e, 4, 0), I, H, dev).cpu().numpy().reshape(-1)
        u = synth.torch_planar(synth.seed_for(cfg, e, 5, 0), I, H, dev).cpu().numpy().reshape(-1)
        gu.append(np.concatenate([g, u]))
        dn.append(synth.torch_planar(synth.seed_for(cfg, e, 6, 0), H, I, dev).cpu().numpy().reshape(-1))
        scales.append([synth.weight_scale(synth.seed_for(cfg, e, p, 1)) for p in (4, 5, 6)])
    router = synth.table_bits_np(synth.seed_for(cfg, 254, 0, 0), E * H, bf16=True)
    block = q.Moe(H, I, K, router, gu, dn, np.array(scales, np.float32), max_batch=B, device=local_rank)
    setup_s = time.time() - t0
    x = np.stack([synth.normal_f32(synth.seed_for(cfg, 253, b, 2), H) for b in range(B)])
    out, ids, w = block.forward(x)
    parity = None
    if not args.no_cpu:
        from oracle import moe as omoe

        same = True
        for b in (0, B - 1):
            want, want_ids, want_w = omoe.forward(x[b], router, gu, dn, np.array(scales, np.float32), H, I, K)
            same = same and list(ids[b]) == list(want_ids) and np.array_equal(w[b].view(np.uint32), want_w.view(np.uint32)) and np.array_equal(out[b].view(np.uint32), want.view(np.uint32))
        parity = {"tokens_checked": 2, "bit_exact": bool(same), "oracle": "composition of the reference's pieces (no reference run exists for this block: parity unpinned)"}
    for _ in range(3):
        block.forward(x)
    t1 = time.perf_counter()
    for _ in range(args.steps):
        block.forward(x)
    e2e_ms = (time.perf_counter() - t1) * 1e3 / args.steps
    ms = block.time_ms(B, max(args.steps, 20))
    weights = B * K * 3 * I * H
    experts_used = len(set(int(i) for i in ids.reshape(-1)))
    block.free()
    return {"shape": "qwen3_30b_a3b FFN block", "hidden": H, "expert_width": I, "experts": E, "top_k": K, "batch": B, "ms_per_block": round(ms, 4), "ms_per_block_host_buffers": round(e2e_ms, 4),
            "weights_streamed": weights, "gweights_per_s": round(weights / (ms * 1e-3) / 1e9, 1), "hbm_frac_of_measured": round(weights * BYTES_PER_WEIGHT / (ms * 1e-3) / 1e9 / measured_peaks()[0], 4),
            "distinct_experts_in_batch": experts_used, "tokens_per_s_ffn_blocks_of_48_layers": round(B / (48 * ms * 1e-3), 1), "setup_s": round(setup_s, 1), "parity_vs_cpu": parity,
            "note": "every (token, expert) pair streams its expert's weights (no sharing between tokens that chose the same expert); one GPU, no expert parallelism"}


def run_moe_ep(args, rank: int, world: int, local_rank: int, dist):
    """The mixture-of-experts block of run_moe with its 128 experts spread over the GPUs (expert parallelism): every rank routes all 16 tokens,
    runs the (token, expert) pairs of the experts it holds and leaves one row of floats per pair; an NCCL all-reduce over the rows viewed as
    int32 adds the ranks' shares (exactly one share of a value is not zero), then every rank weights and adds the pairs in order. Rank 0 also
    runs the whole block alone and compares bits. Wall clock around partial forward + all-reduce + finish, maximum over ranks."""
    import torch

    import quintrit_b200 as q

    dev = torch.device("cuda", local_rank)
    H, I, E, K, B = 2048, 768, 128, 8, 16
    cfg = 4
    if E % world:
        return {"ep_world": world, "skipped": f"{world} ranks do not divide {E} experts"} if rank == 0 else None

    def expert(e):
        g = synth.torch_planar(synth.seed_for(cfg, e, 4, 0), I, H, dev).cpu().numpy().reshape(-1)
        u = synth.torch_planar(synth.seed_for(cfg, e, 5, 0), I, H, dev).cpu().numpy().reshape(-1)
        d = synth.torch_planar(synth.seed_for(cfg, e, 6, 0), H, I, dev).cpu().numpy().reshape(-1)
        return np.concatenate([g, u]), d, [synth.weight_scale(synth.seed_for(cfg, e, p, 1)) for p in (4, 5, 6)]

    per = E // world
    mine = [expert(e) for e in range(rank * per, (rank + 1) * per)]
    router = synth.table_bits_np(synth.seed_for(cfg, 254, 0, 0), E * H, bf16=True)
    x = np.stack([synth.normal_f32(synth.seed_for(cfg, 253, b, 2), H) for b in range(B)])
    block = q.Moe(H, I, K, router, [m[0] for m in mine], [m[1] for m in mine], np.array([m[2] for m in mine], np.float32), max_batch=B, device=local_rank, n_experts=E,
                  expert_first=rank * per)

    def step():
        block.forward_partial(x)
        dist.all_reduce(block.pairs_tensor())
        torch.cuda.synchronize()
        return block.finish()

    out, ids, w = step()
    same = None
    if rank == 0:
        everything = [expert(e) for e in range(E)]
        whole = q.Moe(H, I, K, router, [m[0] for m in everything], [m[1] for m in everything], np.array([m[2] for m in everything], np.float32), max_batch=B, device=local_rank)
        want, want_ids, want_w = whole.forward(x)
        same = bool(np.array_equal(out.view(np.uint32), want.view(np.uint32)) and np.array_equal(ids, want_ids) and np.array_equal(w.view(np.uint32), want_w.view(np.uint32)))
        whole.free()
    for _ in range(3):
        step()
    dist.barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    ms = (time.perf_counter() - t0) * 1e3 / args.steps
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    block.free()
    if rank != 0:
        return None
    return {"shape": "qwen3_30b_a3b FFN block", "ep_world": world, "experts_per_gpu": per, "batch": B, "ms_per_block_host_buffers": round(float(t.item()), 4),
            "exchange": f"NCCL all-reduce of {B * K * H * 4} bytes (the pairs' rows as int32: one share of every value is not zero)", "identical_to_one_gpu": same}


def cpu_decode(shape: str, layers, prompt_len: int, tail: int = 32):
    """The CPU oracle's whole-token decode on the host cores: the seeded prompt is ingested token by token (the reference
    ingests prompts this way, engine.rs:626-631) and the time per token is the mean over the last `tail` positions, i.e. at
    a context of about `prompt_len` tokens. A restatement of the reference's CPU path, not its binary."""
    import oracle

    ctx = (prompt_len + 255) // 256 * 256
    spec = oracle.full_model(shape, "i2_s", ctx, layers=layers)
    m = oracle.Model(spec)
    prompt = synth.prompt_tokens(synth.full_dims(shape)["config"], prompt_len, spec["vocab"])
    times = []
    for pos, tok in enumerate(prompt):
        t0 = time.perf_counter()
        m.forward(int(tok), pos)
        times.append(time.perf_counter() - t0)
    ms = 1e3 * sum(times[-tail:]) / min(tail, len(times))
    return {"shape": shape, "layers": spec["layers"], "context": prompt_len, "tokens_per_s": round(1e3 / ms, 2), "ms_per_token": round(ms, 2),
            "method": f"mean over the last {min(tail, len(times))} of {prompt_len} prompt positions, all host threads", "kind": "port"}


def run_reference(args, rank: int, world: int):
    """--impl reference: the reference's CPU path for the same workload on the host cores (rank 0 only): every step is one
    pass over all projections of the sweep with all host threads. The reference is Rust and cannot be built where this
    runs, so the kernel is its C restatement (kind "port")."""
    if rank != 0:
        return
    threads = pin_to_all_cores()
    sweep = CpuSweep(args.layers)
    for _ in range(max(3, args.warmup)):
        sweep.one_pass(threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        sweep.one_pass(threads)
    ms_per_step = (time.perf_counter() - t0) * 1e3 / args.steps
    value = sweep.weights / (ms_per_step * 1e-3) / 1e9
    by_threads = {str(t): round(sweep.best_of(t), 2) for t in sorted({1, min(4, threads), threads})}
    ceiling = sweep.oracle.stream_read_gbs(1 << 30, threads, 21)
    line = {
        "impl": "reference", "metric": "gemv_gweights_per_s", "value": round(value, 2), "unit": "Gweights/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": round(ms_per_step, 3), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8xternary->int32", "data": "synthetic",
        "config": sweep_config(args.layers, args.gpus, sweep.weights),
        "cpu_baseline": {"value": round(value, 2), "unit": "Gweights/s", "cores": threads, "kind": "port",
                         "sample": f"all {7 * args.layers} projections ({sweep.weights / 1e9:.2f} G weights) per step, {sweep.isa} kernel, threads pinned",
                         "best_of_9_fwd_rev_gweights_per_s_by_threads": by_threads,
                         "host_read_ceiling_gbs": round(ceiling, 1),
                         "share_of_read_ceiling": round(by_threads[str(threads)] * BYTES_PER_WEIGHT / ceiling, 3) if ceiling > 0 else None},
        "e2e": {"value": round(value, 2), "unit": "Gweights/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    if args.gpus == 1 and not args.no_decode:
        del sweep
        try:
            line["decode"] = cpu_decode(args.decode_shape, args.decode_layers, args.prompt)
        except Exception as e:  # the sweep line must still be printed
            line["decode"] = {"error": f"{type(e).__name__}: {e}"}
    print(json.dumps(line), flush=True)


def run_reference_cuda(args, rank: int, world: int, local_rank: int):
    """--impl reference-cuda: the reference's own CUDA projection kernel (quintrit-cuda/kernels/gemv.cu, compiled for sm_100a from the
    reference tree into oracle/_ref by oracle/ref_cuda/Makefile) on the same sweep on this GPU: one launch per projection, as the
    reference's decoder issues them, each with the configuration its device profile picks for that role. Rank 0 only; weights and
    permuted activations resident in HBM; the results of one pass are checked against the CPU kernel's on a sample of projections."""
    if rank != 0:
        return
    from oracle import refcuda

    base = {"impl": "reference-cuda", "metric": "gemv_gweights_per_s", "unit": "Gweights/s", "n_gpus": args.gpus}
    if not refcuda.available():
        print(json.dumps({**base, "unavailable": "oracle/_ref/libqtref_cuda.so is not built (it needs the reference tree at build time)"}), flush=True)
        return
    import torch

    if not torch.cuda.is_available():
        print(json.dumps({**base, "unavailable": "no CUDA device"}), flush=True)
        return
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    l = refcuda.lib()
    role_of = [2, 2, 2, 0, 3, 3, 1]  # q, k, v: the stacked projection's configuration; o: output; gate, up; down
    items = []
    for (layer, p, n, k) in sweep_shapes(args.layers):
        cfg = refcuda.profile_config(role_of[p])
        w = synth.torch_planar(synth.seed_for(CONFIG_ID, layer, p, 0), n, k, dev)
        perm, total = refcuda.permute_activations(activations_for(layer, p, k))
        items.append((cfg, w, n, k, torch.from_numpy(perm).to(dev), torch.tensor([total], dtype=torch.int32, device=dev), torch.zeros(n, dtype=torch.int32, device=dev)))
    weights_total = sum(n * k for _, _, n, k in sweep_shapes(args.layers))
    stream = torch.cuda.current_stream().cuda_stream

    def one_pass():
        for cfg, w, n, k, a, s, o in items:
            rc = l.qtref_gemv_plain_device(cfg, w.data_ptr(), n, k, a.data_ptr(), s.data_ptr(), o.data_ptr(), stream)
            if rc != 0:
                raise RuntimeError(f"the reference kernel failed to launch: CUDA error {rc}")

    one_pass()
    torch.cuda.synchronize()
    checked = 0
    for idx in range(0, len(items), max(1, len(items) // 14)):  # a sample of projections against the CPU kernel
        cfg, w, n, k, a, s, o = items[idx]
        layer, p = divmod(idx, 7)
        import oracle

        want = oracle.gemv_planar(w.cpu().numpy(), n, k, activations_for(layer, p, k))
        if not np.array_equal(o.cpu().numpy(), want):
            raise SystemExit(f"the reference kernel's result of projection {idx} differs from the CPU kernel's")
        checked += 1
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(max(3, args.warmup)):
        one_pass()
    torch.cuda.synchronize()
    sampler.mark_begin()
    t_heat = time.time()
    while time.time() - t_heat < args.preheat:
        for _ in range(10):
            one_pass()
        torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    ev[0].record()
    for i in range(args.steps):
        one_pass()
        ev[i + 1].record()
    torch.cuda.synchronize()
    sampler.mark_end()
    clocks = sampler.stop()
    ms_per_step = ev[0].elapsed_time(ev[-1]) / args.steps
    value = weights_total / (ms_per_step * 1e-3) / 1e9
    peak, peak_kind = measured_peaks()
    achieved = weights_total * BYTES_PER_WEIGHT / (ms_per_step * 1e-3) / 1e9
    print(json.dumps({
        **base, "value": round(value, 1), "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8xternary->int32", "data": "synthetic", "config": sweep_config(args.layers, 1, weights_total),
        "kernel": "the reference's gemv_<config>_plain, one launch per projection (280 per step), configurations of its profile '24sm_24mib' (the nearest to this device by its own rule)",
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4), "traffic": None, "peak_kind": peak_kind},
        "e2e": {"value": round(value, 1), "unit": "Gweights/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": len(items) * args.steps, "clocks": clocks, "parity_vs_cpu": {"projections_checked": checked, "bit_exact": True},
    }), flush=True)


def run_prefill(args, mats, shapes, dev, batch: int = 256, passes: int = 3):
    """The batched projections of a prompt chunk on the tensor cores (quintrit_b200_gemm_i32_device, tcgen05 int8): all projections of the sweep for
    `batch` activation vectors at once, activations resident in HBM. Reported beside the batch-1 sweep: how many tokens' worth of projections a
    second of this kernel gives, its int8 rate, and one projection checked against the batch-1 kernel."""
    import torch

    stream = torch.cuda.current_stream().cuda_stream
    by_cols, outs = {}, {}
    for (_, _, n, k) in shapes:
        if k not in by_cols:
            by_cols[k] = torch.randint(-128, 128, (batch, k), dtype=torch.int8, device=dev)
        if n not in outs:
            outs[n] = torch.zeros((batch, n), dtype=torch.int32, device=dev)

    def one_pass():
        for m, (_, _, n, k) in zip(mats, shapes):
            m.gemm_i32_device(by_cols[k].data_ptr(), batch, outs[n].data_ptr(), stream)

    one_pass()  # makes the two-bit copies of the weights
    torch.cuda.synchronize()
    m0, (_, _, n0, k0) = mats[0], shapes[0]
    m0.gemm_i32_device(by_cols[k0].data_ptr(), batch, outs[n0].data_ptr(), stream)
    torch.cuda.synchronize()
    got = outs[n0][batch - 1].cpu().numpy()
    parity = bool(np.array_equal(got, m0.gemv_i32(by_cols[k0][batch - 1].cpu().numpy())))
    one_pass()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(passes):
        one_pass()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / passes
    weights = sum(n * k for _, _, n, k in shapes)
    tops = 2.0 * weights * batch / (ms * 1e-3) / 1e12
    try:
        bf16 = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"])
    except Exception:
        bf16 = 1590.0
    return {"kernel": "gemm_i8_tcgen05_kernel", "batch": batch, "projections": len(mats), "ms_per_pass": round(ms, 3), "tokens_per_s_projections_only": round(batch / (ms * 1e-3), 1),
            "int8_tops": round(tops, 1), "peak_tops": round(2 * bf16, 1), "peak_kind": "twice the measured dense bf16 rate (int8 runs at twice the bf16 rate on this part)",
            "tensor_frac": round(tops / (2 * bf16), 4), "bit_exact_vs_batch1": parity,
            "note": "every vector has its own activation scale downstream; the integers equal the batch-1 kernel's vector by vector"}


def run_ours(args, rank: int, world: int, local_rank: int):
    import torch

    import quintrit_b200 as q

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist  # noqa: F811

        import datetime

        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=90))  # a rank that fell out does not hang the others forever

    # ---- build the sweep: weights generated on the device, transcoded by the library ----
    t_setup = time.time()
    mats, acts, shapes = [], [], []
    for (l, p, r0, r1, k) in shard_plan(args.layers, rank, world)[0]:
        planar = synth.torch_planar(synth.seed_for(CONFIG_ID, l, p, 0), r1 - r0, k, dev, row0=r0).cpu().numpy()
        mats.append(q.Matrix(planar, r1 - r0, k, device=local_rank))
        acts.append(activations_for(l, p, k))
        shapes.append((l, p, r1 - r0, k))
    torch.cuda.empty_cache()
    plan = q.Plan(mats)
    out_offsets = list(plan.out_offsets)
    weights_local = sum(n * k for _, _, n, k in shapes)
    weights_total = sum(n * k for _, _, n, k in sweep_shapes(args.layers))
    act_host = torch.from_numpy(plan.pack_activations(acts)).pin_memory()
    out_host = torch.zeros(plan.out_total, dtype=torch.int32).pin_memory()
    act_np, out_np = act_host.numpy(), out_host.numpy()
    t_setup = time.time() - t_setup

    stream = torch.cuda.current_stream().cuda_stream

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing: activations already in HBM ----
    plan.run(act_np, out_np)  # also places the activations on the device
    first = out_np.copy()
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(max(3, args.warmup)):
        plan.launch(stream)
    barrier()
    # Warm-up continues for about a second of back-to-back passes, so that the K timed steps that follow without a gap run
    # at the clocks of sustained serving (a cold burst of a few milliseconds runs above them) and the clock samples of this
    # window describe the state the steps were timed in.
    sampler.mark_begin()
    t_heat = time.time()
    heat_steps = 0
    while time.time() - t_heat < args.preheat:
        for _ in range(100):
            plan.launch(stream)
        heat_steps += 100
        torch.cuda.synchronize()
    barrier()
    q.launch_count(reset=True)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    ev[0].record()
    for i in range(args.steps):
        plan.launch(stream)
        ev[i + 1].record()
    barrier()
    sampler.mark_end()
    launches = q.launch_count()
    total_ms = ev[0].elapsed_time(ev[-1])
    per_launch_ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]

    # A further second of back-to-back passes, timed as one block: the long-run rate beside the K-step figure.
    sus0, sus1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_sus = time.time()
    sus_steps = 0
    sus0.record()
    while time.time() - t_sus < 1.0:
        for _ in range(100):
            plan.launch(stream)
        sus_steps += 100
        torch.cuda.synchronize()
    sus1.record()
    torch.cuda.synchronize()
    sustained_ms = sus0.elapsed_time(sus1) / sus_steps
    clocks = sampler.stop()
    clocks["window"] = f"{heat_steps} warm-up passes ({args.preheat:g} s) followed without a gap by the {args.steps} timed steps"

    # ---- end to end through the C ABI with host buffers: H2D activations, kernel, D2H results, every step ----
    for _ in range(2):
        plan.run(act_np, out_np)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        plan.run(act_np, out_np)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    same = bool(np.array_equal(first, out_np))

    if dist is not None:
        t = torch.tensor([total_ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_ms = t.tolist()
        ok = torch.tensor([1 if same else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        same = bool(ok.item())
    decode_tp = None
    h2d_bytes, d2h_bytes = int(plan.act_total), int(plan.out_total * 4)
    prefill = None
    if world == 1 and not args.no_prefill:
        try:
            prefill = run_prefill(args, mats, shapes, dev)
        except Exception as e:  # the sweep line must still be printed
            prefill = {"error": f"{type(e).__name__}: {e}"}
    if dist is not None and not args.no_decode:
        del plan, mats
        torch.cuda.empty_cache()
        try:
            decode_tp = run_decode_tp(args, rank, world, local_rank, dist)
        except Exception as e:  # the sweep line must still be printed
            decode_tp = {"tp_world": world, "error": f"{type(e).__name__}: {e}"}
    moe_ep = None
    if dist is not None and not args.no_moe:
        try:
            moe_ep = run_moe_ep(args, rank, world, local_rank, dist)
        except Exception as e:  # the sweep line must still be printed
            moe_ep = {"ep_world": world, "error": f"{type(e).__name__}: {e}"}
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    ms_per_step = total_ms / args.steps
    value = weights_total / (ms_per_step * 1e-3) / 1e9
    e2e_value = weights_total / (e2e_ms / args.steps * 1e-3) / 1e9
    peak, peak_kind = measured_peaks()
    kernel_ms = statistics.mean(per_launch_ms)
    achieved = weights_local * BYTES_PER_WEIGHT / (kernel_ms * 1e-3) / 1e9
    line = {
        "metric": "gemv_gweights_per_s", "value": round(value, 1), "unit": "Gweights/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8xternary->int32", "data": "synthetic",
        "config": sweep_config(args.layers, world, weights_total),
        "tokens_per_s_gemv_only": round(1e3 / ms_per_step, 1),
        "roofline_nominal_8tbs_frac": round(weights_total * BYTES_PER_WEIGHT / (ms_per_step * 1e-3) / (world * 8e12), 4),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
                     "traffic": int(weights_local * NCU_TRAFFIC_BYTES_PER_WEIGHT), "traffic_source": "ncu capture of the 12-layer case, scaled by weights", "peak_kind": peak_kind, "kernel": "gemv_lut_kernel", "launch_ms": round(kernel_ms, 4),
                     "launch_ms_median": round(statistics.median(per_launch_ms), 4)},
        "e2e": {"value": round(e2e_value, 1), "unit": "Gweights/s", "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
                "ms_per_step": round(e2e_ms / args.steps, 4)},
        "sustained": {"value": round(weights_total / (sustained_ms * 1e-3) / 1e9, 1), "unit": "Gweights/s", "ms_per_step": round(sustained_ms, 4),
                      "steps": sus_steps, "hbm_frac": round(weights_local * BYTES_PER_WEIGHT / (sustained_ms * 1e-3) / 1e9 / peak, 4)},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "deterministic": same,
        "setup_s": round(t_setup, 1),
    }
    if prefill is not None:
        line["prefill"] = prefill
    if decode_tp is not None:
        line["decode"] = decode_tp
    if moe_ep is not None:
        line["moe"] = moe_ep
    if world == 1 and not args.no_decode:
        del plan, mats
        torch.cuda.empty_cache()
        try:
            line["decode"] = run_decode(args, local_rank)
        except Exception as e:  # the sweep line must still be printed
            line["decode"] = {"error": f"{type(e).__name__}: {e}"}
    if world == 1 and not args.no_moe:
        try:
            line["moe"] = run_moe(args, local_rank)
        except Exception as e:
            line["moe"] = {"error": f"{type(e).__name__}: {e}"}
    if world == 1 and not args.no_cpu:
        threads = pin_to_all_cores()
        sweep = CpuSweep(args.layers)
        g = sweep.best_of(threads, reps=5)
        res = [first[o:o + n] for o, (_, _, n, _) in zip(out_offsets, shapes)]
        parity = all(np.array_equal(r, c) for r, c in zip(res, sweep.results()))
        line["cpu_baseline"] = {"value": round(g, 2), "unit": "Gweights/s", "cores": threads, "kind": "port",
                                "sample": f"all {7 * args.layers} projections ({sweep.weights / 1e9:.2f} G weights) per pass, {sweep.isa} kernel, best of 5 passes averaged over forward and reverse order"}
        line["parity_vs_cpu"] = {"projections_checked": len(res), "bit_exact": bool(parity)}
        del sweep
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-cuda"])
    ap.add_argument("--layers", type=int, default=40)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--preheat", type=float, default=1.0, help="seconds of untimed back-to-back passes right before the timed steps")
    ap.add_argument("--no-decode", action="store_true", help="skip the whole-token decode leg")
    ap.add_argument("--no-prefill", action="store_true", help="skip the batched-projection (tensor core) leg")
    ap.add_argument("--decode-only", action="store_true", help="run only the whole-token decode leg and print its object (profiling aid)")
    ap.add_argument("--block-scaled-only", action="store_true", help="run only the block-scaled (Q2_0) projection on the model's shapes (profiling aid)")
    ap.add_argument("--block-scaled-decode", action="store_true", help="run only a whole-token decode of a block-scaled (Q2_0) model of the decode shape (profiling aid)")
    ap.add_argument("--decode-shape", default="falcon3_10b", choices=["falcon3_10b", "bitnet_2b"])
    ap.add_argument("--decode-layers", type=int, default=None, help="fewer layers than the shape has (experiments)")
    ap.add_argument("--moe-only", action="store_true", help="run only the mixture-of-experts block leg and print its object")
    ap.add_argument("--no-moe", action="store_true", help="skip the mixture-of-experts block leg")
    ap.add_argument("--batch-seqs", type=int, default=32, help="sequences of the batched-decode leg (0 skips it)")
    ap.add_argument("--batch-only", action="store_true", help="with --decode-only: run only the batched-decode leg (profiling aid)")
    ap.add_argument("--batch-steps", type=int, default=16, help="greedy steps timed in the batched-decode leg")
    ap.add_argument("--prompt", type=int, default=1024, help="context length at which a decode step is timed")
    ap.add_argument("--parity-full", action="store_true", help="decode the committed full-size fixtures (40 / 30 layers, 1024 + 512 / 512 + 256 tokens) from synthetic GGUF files in every encoding and compare with the CPU oracle's tokens and logits")
    ap.add_argument("--parity-prompt", type=int, default=6, help="prompt tokens of the greedy-token parity check against the CPU oracle")
    ap.add_argument("--parity-new", type=int, default=6, help="greedy tokens compared in that check")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.parity_full:
        import tempfile

        from tests.test_full_parity_gpu import CASES, check_against_fixture  # the same check the GPU test suite runs

        out = []
        with tempfile.TemporaryDirectory() as tmp:
            for model, variant, tables, encoding in CASES:
                if model == args.decode_shape or args.decode_shape == "falcon3_10b" and model == "bitnet_2b":  # the default runs every committed case
                    t0 = time.time()
                    r = check_against_fixture(model, variant, tables, encoding, tmp, device=local_rank)
                    r["seconds"] = round(time.time() - t0, 1)
                    out.append(r)
        print(json.dumps({"parity_full": out}), flush=True)
        return
    if args.block_scaled_only:
        print(json.dumps({"block_scaled": run_block_scaled(args, local_rank)}), flush=True)
        return
    if args.block_scaled_decode:
        print(json.dumps({"block_scaled_decode": run_block_scaled_decode(args, local_rank)}), flush=True)
        return
    if args.moe_only:
        print(json.dumps({"moe": run_moe(args, local_rank)}), flush=True)
        return
    if args.decode_only:
        print(json.dumps({"decode": run_decode(args, local_rank)}), flush=True)
    elif args.impl == "reference":
        run_reference(args, rank, world)
    elif args.impl == "reference-cuda":
        run_reference_cuda(args, rank, world, local_rank)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
