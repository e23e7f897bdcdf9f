"""quant_bench: ``--kernel <name> --size N`` times one device kernel; ``--inference --model m.quant --prompt p``
times generation (tools/bench.cpp:20-185).  Kernel timing: CUDA events on the launching stream, warm-up, an
L2-sized write between timed launches, best and median of ``--iters`` launches; rates are also printed as a
fraction of the copy / GEMM peaks when ``--peaks <json>`` (keys hbm_gbs, bf16_tflops) is given.

Kernels: gemm, gemm_nt_wgrad, gemm_fp8, attention_fwd, attention_bwd, rmsnorm, rmsnorm_bwd, swiglu, rope,
cross_entropy, adamw, paged_decode, sampling, moe_ffn.  ``--comm`` (multi-GPU) times the fused compute+collective kernels
against their NCCL forms (cli/bench_comm.py)."""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import time

from .common import add_int

KERNELS = ("gemm", "gemm_wgrad", "gemm_fp8", "attention_fwd", "attention_bwd", "rmsnorm", "rmsnorm_bwd", "swiglu", "rope",
           "cross_entropy", "adamw", "paged_decode", "sampling", "moe_ffn")


def _build(kernel, n, dev, heads=0, shape=None):
    """Returns (callable, flops, bytes) for one launch of ``kernel`` at problem size ``n``."""
    import torch

    from ..ops import functional as F
    bf = torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)

    def rnd(*shape, dtype=bf, scale=1.0):
        return (torch.randn(*shape, device=dev, generator=g) * scale).to(dtype)
    if kernel == "gemm" and shape:
        # shape = (M, N, K, layout): nt = activations x weight^T (forward), nn = dgrad (weight stored [K, N]),
        # tn = wgrad (both operands stored reduction-major, fp32 accumulate)
        M, N, K, lay = shape
        if lay == "nt":
            a, b, out = rnd(M, K), rnd(N, K), torch.empty((M, N), dtype=bf, device=dev)
            return (lambda: F.gemm(a, b, out=out)), 2.0 * M * N * K, (M * K + N * K + M * N) * 2
        if lay == "nn":
            a, b, out = rnd(M, K), rnd(K, N), torch.empty((M, N), dtype=bf, device=dev)
            return (lambda: F.gemm(a, b, b_mn=True, out=out)), 2.0 * M * N * K, (M * K + N * K + M * N) * 2
        a, b, out = rnd(K, M), rnd(K, N), torch.zeros((M, N), dtype=torch.float32, device=dev)
        return (lambda: F.gemm(a, b, a_mn=True, b_mn=True, out=out, accumulate=True)), 2.0 * M * N * K, (M * K + N * K) * 2 + M * N * 8
    if kernel == "gemm":
        a, b = rnd(n, n), rnd(n, n)
        out = torch.empty((n, n), dtype=bf, device=dev)
        return (lambda: F.gemm(a, b, out=out)), 2.0 * n ** 3, 3 * n * n * 2
    if kernel == "gemm_wgrad":
        a, b = rnd(n, n), rnd(n, n)
        out = torch.zeros((n, n), dtype=torch.float32, device=dev)
        return (lambda: F.gemm(a, b, a_mn=True, b_mn=True, out=out, accumulate=True)), 2.0 * n ** 3, 2 * n * n * 2 + n * n * 8
    if kernel == "gemm_fp8":
        from ..quant import fp8
        qa, sa = fp8.quant_act_1x128(rnd(n, n))
        qb, sb = fp8.quant_weight_128x128(rnd(n, n))
        out = torch.empty((n, n), dtype=bf, device=dev)
        return (lambda: fp8.gemm_fp8(qa, sa, qb, sb, out=out)), 2.0 * n ** 3, 2 * n * n + n * n * 2
    if kernel in ("attention_fwd", "attention_bwd"):
        D, S = 64, n
        H = heads or 8
        B = max(1, (1 << 16) // S)
        qkv = rnd(B * S, 3 * H * D)
        fl = 4.0 * B * H * S * S * D / 2     # causal
        if kernel == "attention_fwd":
            return (lambda: F.attn_fwd(qkv, qkv, qkv, B, S, H, H, D, q_col0=0, k_col0=H * D, v_col0=2 * H * D)), fl, 4 * B * S * H * D * 2
        o, lse = F.attn_fwd(qkv, qkv, qkv, B, S, H, H, D, q_col0=0, k_col0=H * D, v_col0=2 * H * D)
        do, dqkv = rnd(B * S, H * D), torch.empty_like(qkv)
        return (lambda: F.attn_bwd(qkv, qkv, qkv, o, do, lse, dqkv, B, S, H, H, D, q_col0=0, k_col0=H * D, v_col0=2 * H * D)), 2.5 * fl, 8 * B * S * H * D * 2
    if kernel in ("rmsnorm", "rmsnorm_bwd"):
        T, Hd = n * 64, 1024
        x, w = rnd(T, Hd), rnd(Hd)
        if kernel == "rmsnorm":
            return (lambda: F.rmsnorm_fwd(x, w, 1e-5)), 0.0, 2 * T * Hd * 2
        y, h, rstd = F.rmsnorm_fwd(x, w, 1e-5)
        dw = torch.zeros(Hd, dtype=torch.float32, device=dev)
        return (lambda: F.rmsnorm_bwd(x, x, w, rstd, dw)), 0.0, 3 * T * Hd * 2
    if kernel == "swiglu":
        T, Fh = n * 64, 2048
        x = rnd(T, 2 * Fh)
        return (lambda: F.glu_fwd(x, "silu")), 0.0, 3 * T * Fh * 2
    if kernel == "rope":
        S, H, D = 1024, 8, 64
        B = max(1, n * 64 // S)
        x = rnd(B * S, H * D)
        cos, sin = F.rope_tables(D, S, device=dev)
        return (lambda: F.rope_(x, cos, sin, H, D, S)), 0.0, 2 * B * S * H * D * 2
    if kernel == "cross_entropy":
        T, V = n * 16, 32000
        logits = rnd(T, V)
        labels = torch.randint(0, V, (T,), device=dev)
        return (lambda: F.cross_entropy_fwd_bwd(logits, labels)), 0.0, 2 * T * V * 2
    if kernel == "adamw":
        N = n * n * 16
        p, gr = torch.randn(N, device=dev), torch.randn(N, device=dev)
        m, v, lp = torch.zeros(N, device=dev), torch.zeros(N, device=dev), torch.empty(N, dtype=bf, device=dev)
        return (lambda: F.adamw_(p, gr, m, v, lp, 1e-3, 0.9, 0.95, 1e-8, 0.01, 1)), 0.0, N * (4 * 4 + 3 * 4 + 2)
    if kernel == "paged_decode":
        from ..inference.kv_cache import PAGE, PagedKVCache
        B, Hq, Hkv, D, Lctx = 64, 32, 8, 128, n
        pages = B * (Lctx // PAGE)
        kv = PagedKVCache(1, pages, Hkv, D, "bf16", dev)
        kv.k[0].data.normal_()
        kv.v[0].data.normal_()
        bt = torch.arange(pages, device=dev, dtype=torch.int32).view(B, -1)
        sl = torch.full((B,), Lctx, dtype=torch.int32, device=dev)
        q = rnd(B, Hq * D)
        return (lambda: kv.decode(0, q, bt, sl, Hq)), 4.0 * B * Hq * Lctx * D, 2 * B * Lctx * Hkv * D * 2
    if kernel == "sampling":
        from ..inference.sampler import sample
        B, V = max(1, n // 64), 128256
        logits = rnd(B, V, dtype=torch.float32)
        t = torch.full((B,), 0.8, device=dev)
        tk = torch.full((B,), 40, dtype=torch.int32, device=dev)
        tp = torch.full((B,), 0.95, device=dev)
        return (lambda: sample(logits, t, tk, tp, seed=1, step=1)), 0.0, B * V * 4
    if kernel == "moe_ffn":
        from ..ops import moe as M
        T, Hd, Fh, E, k = n * 8, 1024, 512, 16, 2
        x, wr = rnd(T, Hd), rnd(E, Hd, scale=0.1)
        gu, dn = rnd(E, 2 * Fh, Hd, scale=0.05), rnd(E, Hd, Fh, scale=0.05)

        def run():
            with torch.no_grad():
                return M.moe_ffn(x, F.gemm(x, wr, out_dtype=torch.float32), gu, dn, k, True, "silu", 0.0, 0.0)
        return run, 2.0 * T * k * 3 * Hd * Fh, (gu.numel() + dn.numel()) * 2 + 4 * T * Hd * 2
    raise SystemExit(f"Error: unknown kernel '{kernel}' (choices: {', '.join(KERNELS)})")


def time_kernel(fn, iters=20, warmup=5, flush=True):
    """Per-launch milliseconds (list) measured with CUDA events; a 256 MiB write evicts L2 between launches."""
    import torch
    scrub = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(iters):
        if scrub is not None:
            scrub.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1))
    return out


def serve_bench(a):
    """Continuous-batching engine on a random-init preset: B requests of ``prompt_len`` random tokens, ``gen`` new tokens
    each, greedy.  Reports output tokens/s over the whole run, the median time to first token, and the mean decode step."""
    import statistics

    import torch

    from ..inference.engine import EngineConfig, InferenceEngine
    from ..inference.sampler import SamplerConfig
    from ..models.config import preset
    from ..models.dense import DenseModel
    import os
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    symm = None
    if world > 1:                                  # tensor-parallel serving: one process per GPU (torch.distributed.run)
        import torch.distributed as dist

        from ..inference.tp_engine import TPInferenceEngine
        from ..parallel.symm import SymmetricHeap
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        symm = SymmetricHeap(rank, world, dev)
    cfg = preset(a.preset)
    if a.layers > 0:
        cfg.num_layers = a.layers
    if a.tp_shape > 1:
        # one rank's share of a tensor-parallel deployment, alone on this GPU: its heads, kv heads and FFN slice, the
        # replicated embedding / head, and no all-reduce - the compute side of a rank without the peers
        import dataclasses
        assert world == 1 and cfg.num_heads % a.tp_shape == 0 and cfg.ffn_hidden_size % a.tp_shape == 0
        cfg = dataclasses.replace(cfg, num_heads=cfg.num_heads // a.tp_shape, num_kv_heads=max(1, cfg.num_kv_heads // a.tp_shape),
                                  head_dim=cfg.head_dim, ffn_hidden_size=cfg.ffn_hidden_size // a.tp_shape)
    if hasattr(cfg, "num_experts"):
        from ..models.moe import MoEModel
        model = MoEModel(cfg, device=dev, dtype=torch.bfloat16, seed=0)
    else:
        model = DenseModel(cfg, device=dev, dtype=torch.bfloat16, seed=0)
    g = torch.Generator().manual_seed(0)
    if a.load == "baseline5":
        _serve_load(a, cfg, model, rank, world, symm, g)
        if world > 1:
            dist.barrier()
            symm.close()
            dist.destroy_process_group()
        return
    for B in [int(x) for x in a.batch.split(",")]:
        pages = (a.prompt_len + a.gen + 31) // 16 * B + 64
        ecfg = EngineConfig(max_batch=B, num_pages=pages, kv_mode=a.kv, weight_format=a.weights, cuda_graph=not a.no_graph,
                            enable_prefix_cache=False, max_seq_len=min(cfg.max_seq_len, a.prompt_len + a.gen + 16))
        eng = TPInferenceEngine(model, None, ecfg, rank, world, symm) if world > 1 else InferenceEngine(model, None, ecfg)
        greedy = SamplerConfig(temperature=0.0, top_k=0, top_p=1.0)
        for rep in range(3):                       # the first passes build graphs and workspaces and settle the allocator
            prompts = [torch.randint(3, cfg.vocab_size, (a.prompt_len,), generator=g).tolist() for _ in range(B)]
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            reqs = [eng.add_request(p, max_tokens=a.gen, sampling=greedy) for p in prompts]
            d0 = eng.stats.decode_ms
            steps = 0
            while eng.has_pending():
                eng.step()
                steps += 1
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
        out_tokens = sum(len(r.out) for r in reqs)
        rec = {"bench": "serve", "preset": a.preset, "layers": cfg.num_layers, "batch": B, "prompt_len": a.prompt_len, "gen": a.gen, "weights": a.weights or "bf16",
               "kv": a.kv, "tp": world, "cuda_graph": eng.cfg.cuda_graph, "out_tok_s": round(out_tokens / dt, 1),
               "ttft_ms_p50": round(statistics.median((r.t_first - r.t_submit) * 1e3 for r in reqs), 2),
               "decode_ms_per_step": round((eng.stats.decode_ms - d0) / max(1, steps), 3), "total_ms": round(dt * 1e3, 1)}
        if rank == 0:
            print(json.dumps(rec), flush=True)
        del eng
        torch.cuda.empty_cache()
    if world > 1:
        dist.barrier()
        symm.close()
        dist.destroy_process_group()


def _serve_load(a, cfg, model, rank, world, symm, g):
    """Closed-loop load of BASELINE config 5: ``--requests`` (256) requests with prompt lengths uniform in
    [--prompt-min, --prompt-max] (128-2048) and ``--gen`` (256) output tokens each, ``--concurrent`` (64) in flight: a new
    request is submitted the moment one finishes.  Token ids come from the seed.  Reports output tokens/s over the whole
    run and the median / p90 time to first token (submission to first sampled token)."""
    import statistics

    import torch

    from ..inference.engine import EngineConfig, InferenceEngine
    from ..inference.sampler import SamplerConfig
    conc, nreq = a.concurrent, a.requests
    lens = torch.randint(a.prompt_min, a.prompt_max + 1, (nreq,), generator=g).tolist()
    prompts = [torch.randint(3, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    max_len = a.prompt_max + a.gen + 16
    pages = (max_len + 15) // 16 * conc + 64
    ecfg = EngineConfig(max_batch=conc, num_pages=pages, kv_mode=a.kv, weight_format=a.weights, cuda_graph=not a.no_graph,
                        enable_prefix_cache=False, max_seq_len=min(cfg.max_seq_len, max_len))
    if world > 1:
        from ..inference.tp_engine import TPInferenceEngine
        eng = TPInferenceEngine(model, None, ecfg, rank, world, symm)
    else:
        eng = InferenceEngine(model, None, ecfg)
    greedy = SamplerConfig(temperature=0.0, top_k=0, top_p=1.0)
    # warm-up: graphs for the batch buckets, workspaces, allocator
    warm = [eng.add_request(prompts[i % nreq][:256], max_tokens=8, sampling=greedy) for i in range(conc)]
    while eng.has_pending():
        eng.step()
    del warm
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    nxt, live, done = 0, [], []
    d0, steps = eng.stats.decode_ms, 0
    while nxt < nreq or live:
        while nxt < nreq and len(live) < conc:
            live.append(eng.add_request(prompts[nxt], max_tokens=a.gen, sampling=greedy))
            nxt += 1
        eng.step()
        steps += 1
        still = []
        for r in live:
            (done if r.finished else still).append(r)
        live = still
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    out_tokens = sum(len(r.out) for r in done)
    ttft = sorted((r.t_first - r.t_submit) * 1e3 for r in done)
    rec = {"bench": "serve_load", "load": "baseline5", "preset": a.preset, "layers": cfg.num_layers, "requests": nreq,
           "concurrent": conc, "prompt_len": [a.prompt_min, a.prompt_max], "prompt_tokens": sum(lens), "gen": a.gen,
           "weights": a.weights or "bf16", "kv": a.kv, "tp": world, "tp_shape": a.tp_shape, "cuda_graph": eng.cfg.cuda_graph,
           "out_tok_s": round(out_tokens / dt, 1), "ttft_ms_p50": round(statistics.median(ttft), 2),
           "ttft_ms_p90": round(ttft[int(0.9 * (len(ttft) - 1))], 2), "total_s": round(dt, 2), "engine_steps": steps,
           "decode_ms_per_step": round((eng.stats.decode_ms - d0) / max(1, steps), 3),
           "data": "synthetic (seeded token ids; random-init weights)"}
    if rank == 0:
        print(json.dumps(rec), flush=True)


def main(argv=None):
    ap = argparse.ArgumentParser(prog="quant_bench", description="Usage: quant_bench [--kernel <name> --size N] [--inference --model m.quant --prompt p]")
    ap.add_argument("--kernel", default="")
    add_int(ap, "--size", 1024)
    ap.add_argument("--inference", action="store_true")
    ap.add_argument("--serve", action="store_true", help="serving throughput of a random-init preset: out tok/s, TTFT, decode ms/step")
    ap.add_argument("--preset", default="llama-50m")
    ap.add_argument("--batch", default="1,8,64")
    ap.add_argument("--prompt-len", type=int, default=128)
    ap.add_argument("--gen", type=int, default=64)
    ap.add_argument("--weights", default="", help="packed weight format for --serve: int8 | int4 | mxfp8 | fp4 | ternary")
    ap.add_argument("--kv", default="bf16", help="KV cache storage for --serve: bf16 | fp8 | q4")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--layers", type=int, default=0, help="--serve: override the preset's layer count (fits big shapes on one GPU)")
    ap.add_argument("--tp-shape", type=int, default=1, help="--serve on one GPU: serve one rank's share of a TP=N deployment "
                                                             "(heads and FFN divided by N, no collectives)")
    ap.add_argument("--model", default="")
    ap.add_argument("--prompt", default="test")
    add_int(ap, "--iters", 20)
    add_int(ap, "--warmup", 5)
    add_int(ap, "--heads", 0)
    ap.add_argument("--shape", default="", help="gemm only: MxNxK[:nt|nn|tn]")
    ap.add_argument("--peaks", default="")
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--load", default="", help="--serve: 'baseline5' = closed-loop load (256 requests, prompts 128-2048, 256 "
                                               "outputs, 64 concurrent) instead of the fixed-batch sweep")
    ap.add_argument("--requests", type=int, default=256)
    ap.add_argument("--concurrent", type=int, default=64)
    ap.add_argument("--prompt-min", type=int, default=128)
    ap.add_argument("--prompt-max", type=int, default=2048)
    ap.add_argument("--comm", action="store_true", help="fused compute+collective kernels against NCCL + plain kernels "
                                                        "(run under torch.distributed.run; see cli/bench_comm.py)")
    ap.add_argument("--comm-ops", default="all", help="--comm: comma-separated subset of zero2, fsdp, all_reduce, tp_gemm")
    ap.add_argument("--link-gbs", type=float, default=770.0, help="--comm: NVLink bandwidth per direction per GPU, GB/s")
    ap.add_argument("--gemm-tflops", type=float, default=1382.0, help="--comm: sustained bf16 GEMM rate for the roofline")
    ap.add_argument("--zero-mb", type=int, default=256, help="--comm: flat fp32 gradient buffer of the ZeRO-2 step, MiB")
    ap.add_argument("--unit-mb", type=int, default=436, help="--comm: fp32 gradients of one FSDP unit, MiB")
    ap.add_argument("--tokens", type=int, default=8192, help="--comm: rows of the tensor-parallel products")
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--copy-ctas", type=int, default=12)
    a = ap.parse_args(argv)
    if a.comm:
        from .bench_comm import comm_bench
        comm_bench(a)
        return 0
    if a.size <= 0 or a.size > 16384:
        print("Error: --size needs 1..16384", file=sys.stderr)
        return 2
    import torch
    if a.kernel:
        if not torch.cuda.is_available():
            print("Error: kernel benchmarks need a CUDA device", file=sys.stderr)
            return 1
        names = KERNELS if a.kernel == "all" else [a.kernel]
        peaks = json.load(open(a.peaks)) if a.peaks else {}
        for name in names:
            shape = None
            if a.shape:
                dims, _, lay = a.shape.partition(":")
                shape = tuple(int(x) for x in dims.lower().split("x")) + (lay or "nt",)
            fn, flops, nbytes = _build(name, a.size, torch.device("cuda"), a.heads, shape)
            ms = time_kernel(fn, a.iters, a.warmup)
            best, med = min(ms), statistics.median(ms)
            rec = {"kernel": name, "size": a.shape or a.size, "ms_best": round(best, 5), "ms_median": round(med, 5),
                   "gbs": round(nbytes / best / 1e6, 1), "tflops": round(flops / best / 1e9, 2)}
            if peaks:
                rec["frac_hbm_of_measured"] = round(rec["gbs"] / peaks["hbm_gbs"], 3)
                if flops:
                    rec["frac_bf16_of_measured"] = round(rec["tflops"] / peaks["bf16_tflops"], 3)
            print(json.dumps(rec) if a.json else "  ".join(f"{k}={v}" for k, v in rec.items()), flush=True)
    if a.serve:
        serve_bench(a)
    if a.inference:
        from ..inference.engine import EngineConfig, InferenceEngine
        from ..inference.sampler import SamplerConfig
        from ..quant import codec
        from .common import load_tokenizer, model_dtype, pick_device
        dev = pick_device()
        model = codec.load_model(a.model, device=dev, dtype=model_dtype(dev))
        eng = InferenceEngine(model, load_tokenizer(a.model), EngineConfig(num_pages=1024))
        t0 = time.perf_counter()
        text, st = eng.generate_with_stats(a.prompt, min(64, model.cfg.max_seq_len - 8), SamplerConfig(0.0))
        dt = time.perf_counter() - t0
        print(f"inference: {st.generated_tokens} tokens in {dt * 1e3:.1f} ms ({st.generated_tokens / max(dt, 1e-9):.1f} tok/s, ttft {st.ttft_ms:.2f} ms)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
