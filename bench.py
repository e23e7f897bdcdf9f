#!/usr/bin/env python
"""Headline benchmark: training throughput (tokens/s).

Default configuration: the ~50M-parameter Llama-style decoder with ZeRO-2 data parallelism on 1/2/4/8 B200 (bf16
compute, fp32 master weights, AdamW, seq 1024, global batch 64, uniform-random token ids from a seed, random-init weights).
``--config llama3-8b-fsdp-tp2``: Llama-3-8B shape with ZeRO-3 over the dp ranks x tensor parallel 2 (seq 4096, one
sequence per GPU) on 2, 4 or 8 GPUs.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --config llama3-8b-fsdp-tp2 --steps 5 --warmup 3

Two timed regions, both device-timed with CUDA events, barrier + synchronize on both sides, max over
ranks: (1) K steps on device-resident batches -> "value"; (2) K steps through the public
``TrainEngine.train_step`` with a fresh pinned-host batch copied in and the loss read back every
step -> "e2e".  Rank 0 prints one JSON line.
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

MODEL = "llama-50m (8L d512 8h ff1408 SwiGLU RMSNorm RoPE vocab32000 tied)"
GLOBAL_BATCH = 64
SEQ = 1024


def cpu_inference_config(args):
    """BASELINE config 1, the one configuration the reference can run too: GPT-2-small-shaped decoder on the CPU (12 layers,
    d_model 768, 12 heads, d_ff 3072, GELU, vocab 50257, fp32, seeded random init), batch 1, 32 uniform-random prompt tokens,
    64 greedy tokens.  ``--impl reference`` runs the unmodified reference library through its Generator (harness
    baseline/ref_gpt2_cpu.cpp, built by baseline/build_reference.sh into baseline/_ref); ours runs the repository's CPU
    path (pre-LayerNorm + learned positions, the paged engine) through InferenceEngine.  Wall-clock, whole generation."""
    import time
    here = os.path.dirname(os.path.abspath(__file__))
    if args.impl == "reference":
        exe = os.path.join(here, "baseline", "_ref", "bin", "ref_gpt2_cpu")
        if not os.path.exists(exe):
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/bin/ref_gpt2_cpu is not built; run "
                                                                  "baseline/build_reference.sh"}))
            return 0
        r = subprocess.run([exe, "12", "64"], capture_output=True, text=True, timeout=1800)
        print(r.stdout.strip().splitlines()[-1] if r.returncode == 0 and r.stdout.strip() else
              json.dumps({"impl": "reference", "unavailable": f"harness exited {r.returncode}: {r.stderr[-200:]}"}))
        return 0
    import torch
    from transformers_fusion_b200.inference.engine import EngineConfig, InferenceEngine
    from transformers_fusion_b200.inference.sampler import SamplerConfig
    from transformers_fusion_b200.models.config import preset
    from transformers_fusion_b200.models.dense import DenseModel
    cfg = preset("gpt2-small")
    model = DenseModel(cfg, device="cpu", dtype=torch.float32, seed=0)
    eng = InferenceEngine(model, None, EngineConfig(max_batch=1, num_pages=16, enable_prefix_cache=False, max_seq_len=128))
    g = torch.Generator().manual_seed(0)
    greedy = SamplerConfig(temperature=0.0, top_k=0, top_p=1.0)
    best = None
    for rep in range(max(2, min(args.steps, 5))):
        prompt = torch.randint(0, cfg.vocab_size, (32,), generator=g).tolist()
        t0 = time.perf_counter()
        req = eng.add_request(prompt, max_tokens=64, sampling=greedy)
        while eng.has_pending():
            eng.step()
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
        n = len(req.out)
    print(json.dumps({"impl": "ours", "metric": "generated_tokens_per_s", "value": n / best, "unit": "tokens/s", "seconds": best,
                      "prompt_tokens": 32, "new_tokens": n, "layers": cfg.num_layers, "dtype": "fp32", "device": "cpu",
                      "threads": torch.get_num_threads(), "higher_is_better": True,
                      "config": {"model": "gpt2-small shape (12L d768 12h ff3072 GELU pre-LayerNorm learned positions vocab50257)",
                                 "batch": 1, "prompt": 32, "decode": "greedy, 64 new tokens"}}))
    return 0


def reference_arm(args):
    """The reference is a CPU-only C++/CMake project with no Python packaging: the prescribed
    ``pip install --target baseline/_ref <reference tree>`` fails ("neither setup.py nor
    pyproject.toml found"), and its own trainer runs ~8 tokens/s at this model size on one core, so a
    single 65,536-token step would take hours."""
    print(json.dumps({"impl": "reference",
                      "unavailable": "reference is a CPU-only C++ CMake project without setup.py/pyproject.toml: "
                                     "pip install into baseline/_ref fails; it has no GPU or multi-process "
                                     "training path for this config"}))
    return 0


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); pw.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm), "reasons": sorted(reasons)}


def torch_library_arm(cfg, world, rank, dev, local_batch, seq, steps, warmup, dist):
    """The library baseline of the same training step: the same architecture written with stock PyTorch modules
    (cuBLAS matmuls, the library's fused scaled-dot-product attention, autograd, bf16 autocast over fp32 master weights,
    torch.optim.AdamW(fused=True)) and, on more than one GPU, DistributedDataParallel over NCCL.  None of this repo's
    kernels run here.  Returns tokens/s over all ranks (device-timed, max over ranks)."""
    import torch
    import torch.nn as nn
    import torch.nn.functional as TF
    H, D, Hq, Hkv, Fh = cfg.hidden_size, cfg.head_dim, cfg.num_heads, cfg.num_kv_heads, cfg.ffn_hidden_size

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.n1, self.n2 = nn.RMSNorm(H, eps=cfg.norm_eps), nn.RMSNorm(H, eps=cfg.norm_eps)
            self.qkv = nn.Linear(H, (Hq + 2 * Hkv) * D, bias=False)
            self.o = nn.Linear(Hq * D, H, bias=False)
            self.gu = nn.Linear(H, 2 * Fh, bias=False)
            self.down = nn.Linear(Fh, H, bias=False)

        def forward(self, x, cos, sin):
            B, S, _ = x.shape
            q, k, v = self.qkv(self.n1(x)).split([Hq * D, Hkv * D, Hkv * D], -1)
            q, k, v = (t.view(B, S, -1, D).transpose(1, 2) for t in (q, k, v))

            def rot(t):
                t1, t2 = t[..., : D // 2], t[..., D // 2:]
                return torch.cat([t1 * cos - t2 * sin, t2 * cos + t1 * sin], -1)
            a = TF.scaled_dot_product_attention(rot(q), rot(k), v, is_causal=True, enable_gqa=Hq != Hkv)
            x = x + self.o(a.transpose(1, 2).reshape(B, S, Hq * D))
            g, u = self.gu(self.n2(x)).chunk(2, -1)
            return x + self.down(TF.silu(g) * u)

    class LM(nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = nn.Embedding(cfg.vocab_size, H)
            self.blocks = nn.ModuleList(Block() for _ in range(cfg.num_layers))
            self.norm = nn.RMSNorm(H, eps=cfg.norm_eps)
            inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2).float() / D))
            ang = torch.outer(torch.arange(seq).float(), inv)
            self.register_buffer("cos", ang.cos()[None, None].to(torch.bfloat16))
            self.register_buffer("sin", ang.sin()[None, None].to(torch.bfloat16))

        def forward(self, ids, labels):
            x = self.emb(ids)
            for b in self.blocks:
                x = b(x, self.cos, self.sin)
            logits = TF.linear(self.norm(x), self.emb.weight)
            return TF.cross_entropy(logits.view(-1, logits.shape[-1]).float(), labels.reshape(-1))
    torch.manual_seed(0)
    model = LM().to(dev)
    for prm in model.parameters():
        if prm.dim() >= 2:
            nn.init.normal_(prm, std=cfg.init_std)
    net = nn.parallel.DistributedDataParallel(model, device_ids=[dev.index], gradient_as_bucket_view=True) if world > 1 else model
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
    g = torch.Generator().manual_seed(99 + rank)
    ids = [torch.randint(0, cfg.vocab_size, (local_batch, seq), generator=g).to(dev) for _ in range(4)]

    def step(i):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = net(ids[i % 4], torch.roll(ids[i % 4], -1, 1))
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        opt.zero_grad(set_to_none=True)
    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    del net, model, opt
    torch.cuda.empty_cache()
    return local_batch * world * seq * steps / (float(ms) / 1e3)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "nccl"])
    ap.add_argument("--config", default="llama-50m-zero2", choices=["llama-50m-zero2", "llama3-8b-fsdp-tp2", "mixtral-8x7b-ep", "gpt2-small-cpu"],
                    help="llama-50m-zero2: ~50M Llama, ZeRO-2 data parallel, seq 1024, global batch 64 (the default; runs on "
                         "1/2/4/8 GPUs).  llama3-8b-fsdp-tp2: Llama-3-8B shape, ZeRO-3 over dp x tensor parallel 2, seq 4096, "
                         "one sequence per GPU (2, 4 or 8 GPUs).  gpt2-small-cpu: GPT-2-small-shaped greedy generation on the CPU "
                         "(32 prompt + 64 new tokens), the configuration the reference's own build can run as well")
    ap.add_argument("--capacity-factor", type=float, default=2.0,
                    help="mixtral-8x7b-ep: expert buffer rows per rank as a multiple of the balanced load")
    ap.add_argument("--no-graph", action="store_true", help="launch kernels eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-baseline", action="store_true", help="skip the library-baseline arm that fills vs_baseline")
    ap.add_argument("--model", default="llama-50m")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (stated in the config line)")
    ap.add_argument("--tp", type=int, default=2, help="llama3-8b-fsdp-tp2: tensor-parallel degree")
    ap.add_argument("--kernel-table", default="", metavar="FILE",
                    help="llama3-8b-fsdp-tp2: after the timed steps run one more step under the PyTorch profiler and write "
                         "rank 0's per-kernel table to FILE (shares of a step; never the source of a reported number)")
    ap.add_argument("--gather", default="auto", choices=["auto", "prefetch", "fused"],
                    help="llama3-8b-fsdp-tp2: ZeRO-3 weight gather by a prefetching kernel on a side stream, or inside the "
                         "GEMM that first uses the weight")
    ap.add_argument("--global-batch", type=int, default=GLOBAL_BATCH,
                    help="sequences per step over all ranks (the headline configuration is the default; other values are "
                         "for studying one rank's share of a larger job on a single GPU)")
    args = ap.parse_args(argv)
    if args.config == "gpt2-small-cpu":
        return cpu_inference_config(args)
    if args.impl == "reference":
        return reference_arm(args)
    if args.config == "llama3-8b-fsdp-tp2":
        return main_sharded(args)
    if args.config == "mixtral-8x7b-ep":
        return main_ep(args)

    import torch
    import torch.distributed as dist

    from transformers_fusion_b200.models.config import preset
    from transformers_fusion_b200.models.dense import DenseModel
    from transformers_fusion_b200.ops import _lib
    from transformers_fusion_b200.trainer.engine import TrainEngine

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if rank == 0:
            print(f"bench.py: --gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run", file=sys.stderr)
        if world == 1 and args.gpus > 1:
            return 2
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    symm = None
    comm = "none"
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        comm = "nccl" if args.impl == "nccl" else "fused"
        if comm == "fused":
            from transformers_fusion_b200.parallel.symm import SymmetricHeap
            symm = SymmetricHeap(rank, world, dev)

    cfg = preset(args.model)
    if args.layers > 0:
        cfg.num_layers = args.layers
    global_batch = args.global_batch
    assert global_batch % world == 0
    local_batch = global_batch // world
    graph = not args.no_graph

    def make_engine(comm_):
        m = DenseModel(cfg, device=dev, dtype=torch.bfloat16, seed=0)
        return TrainEngine(m, lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, max_grad_norm=1.0, zero_stage=2,
                           comm=comm_, cuda_graph=graph, symm=symm if comm_ == "fused" else None)
    engine = make_engine(comm)

    # synthetic data: uniform token ids from a seed, a different pinned-host batch every step
    g = torch.Generator().manual_seed(1234 + rank)
    n_host = 8
    host_ids = [torch.randint(0, cfg.vocab_size, (local_batch, SEQ), generator=g).pin_memory() for _ in range(n_host)]
    host_lab = [torch.roll(t, -1, 1).pin_memory() for t in host_ids]
    dev_ids = [t.to(dev) for t in host_ids]
    dev_lab = [t.to(dev) for t in host_lab]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    launches_per_step = [0]
    eng_ref = [engine]

    def dev_step(i):
        eng_ref[0].step(dev_ids[i % n_host], dev_lab[i % n_host])

    last_loss = [0.0]

    pending = [None]

    def e2e_step(i):
        # public API, one step late on the read: enqueue step i from pinned host memory, then read the loss of step i - 1
        # (its device-to-host copy is behind an event); the last step's loss is read before the timed region closes
        h = engine.train_step_async(host_ids[i % n_host], host_lab[i % n_host])
        if pending[0] is not None:
            last_loss[0] = pending[0].value()
        pending[0] = h
        if i == args.steps - 1:
            last_loss[0] = h.value()
            pending[0] = None

    W = max(3, args.warmup)
    c0 = _lib.LAUNCHES[0]
    for i in range(W):
        dev_step(i)
    torch.cuda.synchronize()
    _lib.check_status(dev)
    launches_per_step[0] = engine.launches_per_step if engine.launches_per_step else (_lib.LAUNCHES[0] - c0) // W

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms_dev = timed(dev_step, args.steps)
    ms_e2e = timed(e2e_step, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    _lib.check_status(dev)

    tokens = global_batch * SEQ * args.steps
    value = tokens / (ms_dev / 1e3)
    e2e = tokens / (ms_e2e / 1e3)

    # ---- baselines, same process, same box, after the headline numbers are in
    base = {}
    if not args.no_baseline and args.impl == "ours":
        bsteps = max(3, min(args.steps, 10))
        if world > 1:
            # this repo's kernels with NCCL collectives in place of the fused reduce-scatter / AdamW / all-gather kernels
            # (same CUDA-graph setting): isolates what the fused communication path is worth
            del engine
            eng_ref[0] = None
            torch.cuda.empty_cache()
            try:
                eng_ref[0] = make_engine("nccl")
                for i in range(3):
                    dev_step(i)
                base["nccl_arm_tokens_per_s"] = global_batch * SEQ * bsteps / (timed(dev_step, bsteps) / 1e3)
            except Exception as ex:          # graph capture of NCCL can be refused by the library; say so rather than guess
                base["nccl_arm_error"] = f"{type(ex).__name__}: {ex}"[:200]
            eng_ref[0] = None
            torch.cuda.empty_cache()
        try:
            base["torch_library_tokens_per_s"] = torch_library_arm(cfg, world, rank, dev, local_batch, SEQ, bsteps, 3, dist)
        except Exception as ex:
            base["torch_library_error"] = f"{type(ex).__name__}: {ex}"[:200]
    lib_tps = base.get("torch_library_tokens_per_s")
    if rank == 0:
        out = {
            "metric": "train_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": W, "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": (value / lib_tps) if lib_tps else None, "dtype": "bf16",
            "data": "synthetic (seeded uniform token ids; random-init weights)",
            "impl": "ours" if args.impl == "ours" else "ours-nccl-baseline",
            "config": {"model": MODEL if args.layers <= 0 else MODEL + f" [layers overridden to {args.layers}]",
                       "global_batch": global_batch, "seq_len": SEQ,
                       "parallelism": f"dp{world}-zero2" if world > 1 else "single",
                       "optimizer": "AdamW fp32 master", "comm": comm, "cuda_graph": graph,
                       "l2": "per-step working set (activations + logits, several GB) exceeds the 126 MB L2; "
                             "no explicit flush",
                       "baseline": "vs_baseline = value / the library baseline measured in this process on this box: the same "
                                   "architecture in stock PyTorch (cuBLAS, fused SDPA, autograd, bf16 autocast, fused AdamW, DDP "
                                   "over NCCL); the reference itself publishes no number and cannot run this config",
                       **{k: (round(v, 1) if isinstance(v, float) else v) for k, v in base.items()},
                       "vs_nccl_arm": (value / base["nccl_arm_tokens_per_s"]) if base.get("nccl_arm_tokens_per_s") else None},
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": int(2 * local_batch * SEQ * 8), "d2h_bytes_per_step": 4,
                    "last_loss": last_loss[0]},
            "gpu_launches": int(launches_per_step[0] * args.steps),
            "clocks": clocks,
            "model_tflops_per_gpu": cfg.flops_per_token(SEQ) * value / world / 1e12,
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


def main_ep(args):
    """BASELINE config 4: Mixtral-8x7B shape (d4096, 32q/8kv heads, 8 SwiGLU experts of d_ff 14336, top-2 router with
    load-balance loss 0.01, vocab 32000), expert parallel over all ranks (8 / N experts per rank per layer), seq 4096, one
    sequence per GPU, bf16 experts (the block-scaled fp8 expert GEMM of this repository is slower than its bf16 GEMM and is
    not used here), fused dispatch / combine over NVLink peer memory, fused AdamW.  ``--layers`` trims the depth so that
    fp32 AdamW state of the local experts fits (stated in the config line)."""
    import torch
    import torch.distributed as dist

    from transformers_fusion_b200.models.config import preset
    from transformers_fusion_b200.models.moe import MoEModel
    from transformers_fusion_b200.ops import _lib
    from transformers_fusion_b200.parallel.ep_model import EPTrainer, attach_expert_parallel
    from transformers_fusion_b200.parallel.symm import SymmetricHeap
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus or world < 2:
        print("bench.py: --config mixtral-8x7b-ep needs --gpus == WORLD_SIZE >= 2 (torch.distributed.run)", file=sys.stderr)
        return 2
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    cfg = preset("mixtral-8x7b")
    cfg.expert_fp8 = False
    cfg.num_layers = args.layers if args.layers > 0 else 8
    seq = 4096
    El = cfg.num_experts // world
    # build only this rank's experts: the block constructor is given the local expert count, the router keeps all 8 outputs
    full_E = cfg.num_experts
    model = MoEModel(cfg, device=dev, dtype=torch.bfloat16, seed=None)
    g = torch.Generator(device=dev).manual_seed(7)
    with torch.no_grad():
        for name, prm in model.named_parameters():
            if prm.dim() >= 2:
                prm.copy_((torch.randn(prm.shape, device=dev, generator=g) * cfg.init_std).to(prm.dtype))
            else:
                prm.fill_(1.0)
    symm = SymmetricHeap(rank, world, dev)
    experts = attach_expert_parallel(model, symm, rank, world, seq, capacity_factor=args.capacity_factor)
    torch.cuda.empty_cache()
    tr = EPTrainer(model, experts, lr=3e-4, weight_decay=0.1, max_grad_norm=1.0)
    gh = torch.Generator().manual_seed(1234 + rank)
    n_host = 4
    host_ids = [torch.randint(0, cfg.vocab_size, (1, seq), generator=gh).pin_memory() for _ in range(n_host)]
    host_lab = [torch.roll(t, -1, 1).pin_memory() for t in host_ids]
    dev_ids, dev_lab = [t.to(dev) for t in host_ids], [t.to(dev) for t in host_lab]

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())
    last_loss = [0.0]

    def dev_step(i):
        last_loss[0] = tr.train_step(dev_ids[i % n_host], dev_lab[i % n_host])

    def e2e_step(i):
        ids = host_ids[i % n_host].to(dev, non_blocking=True)
        lab = host_lab[i % n_host].to(dev, non_blocking=True)
        last_loss[0] = tr.train_step(ids, lab)               # returns the loss as a host float: one read per step
    W = max(3, args.warmup)
    c0 = _lib.LAUNCHES[0]
    for i in range(W):
        dev_step(i)
    torch.cuda.synchronize()
    _lib.check_status(dev)
    launches = (_lib.LAUNCHES[0] - c0) // W
    torch.cuda.reset_peak_memory_stats(dev)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms_dev = timed(dev_step, args.steps)
    ms_e2e = timed(e2e_step, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    _lib.check_status(dev)
    peak = torch.tensor([float(torch.cuda.max_memory_allocated(dev))], device=dev)
    dist.all_reduce(peak, op=dist.ReduceOp.MAX)
    tokens = world * seq * args.steps
    value, e2e = tokens / (ms_dev / 1e3), tokens / (ms_e2e / 1e3)
    H, Fe, k = cfg.hidden_size, cfg.expert_hidden_size, cfg.top_k
    attn_params = H * (cfg.num_heads + 2 * cfg.num_kv_heads) * cfg.head_dim + H * cfg.num_heads * cfg.head_dim
    flops_tok = 6 * (cfg.num_layers * (attn_params + k * 3 * H * Fe + full_E * H) + cfg.vocab_size * H) + \
        12 * cfg.num_layers * cfg.num_heads * cfg.head_dim * seq // 2
    # rows that cross NVLink per layer and direction: each token goes to top-2 experts, (W - 1) / W of them remote
    a2a_bytes = 2 * 2 * seq * k * H * 2 * (world - 1) / world * cfg.num_layers      # dispatch + combine, forward + backward
    if rank == 0:
        out = {
            "metric": "train_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": W,
            "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (seeded uniform token ids; random-init weights)", "impl": "ours",
            "config": {"model": f"mixtral-8x7b shape ({cfg.num_layers} of 32 layers, d4096 32q/8kv heads, 8 experts ff14336 top-2, aux 0.01, "
                                f"vocab32000); experts in bf16",
                       "global_batch": world, "seq_len": seq, "parallelism": f"ep{world} ({El} expert(s) per rank per layer), "
                                                                           "replicated attention / router data parallel",
                       "optimizer": "AdamW fp32 master (fused)", "comm": "fused dispatch / combine over peer memory; NCCL all-reduce "
                                                                         "for the replicated gradients",
                       "capacity_factor": args.capacity_factor, "cuda_graph": False,
                       "l2": "per-step working set (tens of GB) exceeds the 126 MB L2; no explicit flush",
                       "peak_allocated_gb_max_rank": round(float(peak) / 2 ** 30, 2),
                       "all_to_all_gb_per_step_per_rank": round(a2a_bytes / 1e9, 2),
                       "baseline": "none: the reference cannot run this configuration and publishes no number"},
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps, "h2d_bytes_per_step": int(2 * seq * 8),
                    "d2h_bytes_per_step": 4, "last_loss": float(last_loss[0])},
            "gpu_launches": int(launches * args.steps), "clocks": clocks,
            "model_tflops_per_gpu": flops_tok * value / world / 1e12,
        }
        print(json.dumps(out))
    dist.barrier()
    symm.close()
    dist.destroy_process_group()
    return 0


def main_sharded(args):
    """BASELINE config 3: Llama-3-8B shape, ZeRO-3 (FSDP) over the dp ranks x tensor parallel ``--tp``, seq 4096, one
    sequence per GPU, bf16 compute with fp32 master weights and AdamW, synthetic tokens, random-init weights."""
    import torch
    import torch.distributed as dist

    from transformers_fusion_b200.models.config import preset
    from transformers_fusion_b200.ops import _lib
    from transformers_fusion_b200.parallel.launch import init_parallel
    from transformers_fusion_b200.parallel.sharded import Mesh, ShardedEngine
    from transformers_fusion_b200.parallel.symm import SymmetricHeap

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus or world < 2:
        print(f"bench.py: --config llama3-8b-fsdp-tp2 needs --gpus == WORLD_SIZE >= 2 (torch.distributed.run)", file=sys.stderr)
        return 2
    tp = min(args.tp, world)
    st = init_parallel(tp=tp)
    rank, dev = st.rank, st.device
    cfg = preset("llama-3-8b")
    if args.layers > 0:
        cfg.num_layers = args.layers
    seq = 4096
    comm = "nccl" if args.impl == "nccl" else "fused"
    mesh = Mesh(st.dp_rank, st.dp, st.tp_rank, st.tp, st.dp_group, st.tp_group, None)
    T = tp * seq                                    # tokens of one dp group per step: one sequence per GPU

    def make_engine(comm_):
        heaps = [None, None]
        if comm_ == "fused":
            if st.dp > 1:
                heaps[0] = SymmetricHeap(st.dp_rank, st.dp, dev, group=st.dp_group)
            if st.tp > 1:
                heaps[1] = SymmetricHeap(st.tp_rank, st.tp, dev, group=st.tp_group)
        e = ShardedEngine.from_config(cfg, mesh, dev, seed=0, comm=comm_, dp_heap=heaps[0], tp_heap=heaps[1], lr=3e-4,
                                      betas=(0.9, 0.95), weight_decay=0.1, max_grad_norm=1.0, max_tokens=T,
                                      gather=args.gather)
        return e, heaps
    engine, heaps = make_engine(comm)
    g = torch.Generator().manual_seed(1234 + st.dp_rank)      # the tp ranks of one dp group see the same batch
    n_host = 4
    host_ids = [torch.randint(0, cfg.vocab_size, (tp, seq), generator=g).pin_memory() for _ in range(n_host)]
    host_lab = [torch.roll(t, -1, 1).pin_memory() for t in host_ids]
    dev_ids = [t.to(dev) for t in host_ids]
    dev_lab = [t.to(dev) for t in host_lab]

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())
    eng_ref = [engine]
    last = [None]

    def dev_step(i):
        last[0] = eng_ref[0].train_step(dev_ids[i % n_host], dev_lab[i % n_host])

    loss_host = torch.zeros(1).pin_memory()
    last_loss = [0.0]

    def e2e_step(i):
        ids = host_ids[i % n_host].to(dev, non_blocking=True)
        lab = host_lab[i % n_host].to(dev, non_blocking=True)
        loss = eng_ref[0].train_step(ids, lab)
        loss_host.copy_(loss.detach().reshape(1).float())        # the step's loss, read on the host every step
        last_loss[0] = float(loss_host[0])
    W = max(3, args.warmup)
    c0 = _lib.LAUNCHES[0]
    for i in range(W):
        dev_step(i)
    torch.cuda.synchronize()
    _lib.check_status(dev)
    launches = (_lib.LAUNCHES[0] - c0) // W
    torch.cuda.reset_peak_memory_stats(dev)
    sampler = ClockSampler(st.local_rank)
    if rank == 0:
        sampler.start()
    ms_dev = timed(dev_step, args.steps)
    ms_e2e = timed(e2e_step, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    _lib.check_status(dev)
    peak = torch.tensor([float(torch.cuda.max_memory_allocated(dev))], device=dev)
    dist.all_reduce(peak, op=dist.ReduceOp.MAX)
    if args.kernel_table:
        from torch.profiler import ProfilerActivity, profile
        barrier()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            dev_step(0)
            torch.cuda.synchronize()
        if rank == 0:
            with open(args.kernel_table, "w") as f:
                f.write(prof.key_averages().table(sort_by="cuda_time_total", row_limit=40, max_name_column_width=70))
        barrier()
    memp = engine.memory_profile()
    heap_bytes = sum(b.nbytes for h in heaps if h is not None for b in h.buffers)
    global_tokens = st.dp * T
    tokens = global_tokens * args.steps
    value, e2e = tokens / (ms_dev / 1e3), tokens / (ms_e2e / 1e3)
    base = {}
    if not args.no_baseline and comm == "fused":
        # the same engine with every fused piece replaced by the NCCL collective + plain kernel (the library baseline of
        # this configuration; a stock-PyTorch FSDP + tensor-parallel 8B job is not part of this repository)
        bsteps = max(3, min(args.steps, 5))
        del engine
        eng_ref[0] = None
        for h in heaps:
            if h is not None:
                h.close()
        torch.cuda.empty_cache()
        try:
            eng_ref[0], _ = make_engine("nccl")
            for i in range(3):
                dev_step(i)
            base["nccl_arm_tokens_per_s"] = global_tokens * bsteps / (timed(dev_step, bsteps) / 1e3)
        except Exception as ex:
            base["nccl_arm_error"] = f"{type(ex).__name__}: {ex}"[:200]
    nccl_tps = base.get("nccl_arm_tokens_per_s")
    if rank == 0:
        out = {
            "metric": "train_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": W,
            "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / nccl_tps) if nccl_tps else None, "dtype": "bf16",
            "data": "synthetic (seeded uniform token ids; random-init weights drawn on the device per tensor)",
            "impl": "ours" if comm == "fused" else "ours-nccl-baseline",
            "config": {"model": f"llama-3-8b shape ({cfg.num_layers}L d4096 32q/8kv heads ff14336 SwiGLU RMSNorm RoPE 5e5 vocab128256)"
                                + (f" [layers overridden to {args.layers}]" if args.layers > 0 else ""),
                       "global_batch": world, "seq_len": seq, "parallelism": f"fsdp(zero3)-dp{st.dp} x tp{st.tp} + sequence parallel",
                       "optimizer": "AdamW fp32 master (sharded)", "comm": comm, "cuda_graph": False,
                       "l2": "per-step working set (tens of GB) exceeds the 126 MB L2; no explicit flush",
                       "baseline": "vs_baseline = value / the same engine with NCCL collectives + plain kernels in place of the "
                                   "fused ones, measured in this process; the reference cannot run this config",
                       **{k: (round(v, 1) if isinstance(v, float) else v) for k, v in base.items()},
                       "peak_allocated_gb_max_rank": round(float(peak) / 2 ** 30, 2),
                       "symmetric_heap_gb": round(heap_bytes / 2 ** 30, 2),
                       "state_gb": {k: round(v / 2 ** 30, 2) for k, v in memp.items()}},
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": int(2 * tp * seq * 8), "d2h_bytes_per_step": 4, "last_loss": last_loss[0]},
            "gpu_launches": int(launches * args.steps),
            "clocks": clocks,
            "model_tflops_per_gpu": cfg.flops_per_token(seq) * value / world / 1e12,
        }
        print(json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
