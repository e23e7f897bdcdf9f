"""Worker for the tensor-parallel serving test: every rank runs TPInferenceEngine on the same prompts; rank 0 also runs the
single-process engine on the full model and the outputs are compared.  argv: <out_dir> <cpu|cuda>."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from transformers_fusion_b200.inference.engine import EngineConfig, InferenceEngine  # noqa: E402
from transformers_fusion_b200.inference.sampler import SamplerConfig  # noqa: E402
from transformers_fusion_b200.inference.tp_engine import TPInferenceEngine  # noqa: E402
from transformers_fusion_b200.models.config import TransformerConfig  # noqa: E402
from transformers_fusion_b200.models.dense import DenseModel  # noqa: E402


def main():
    out_dir, where = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    symm = None
    if where == "cuda":
        dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", device_id=dev)
        from transformers_fusion_b200.parallel.symm import SymmetricHeap
        symm = SymmetricHeap(rank, world, dev)
        dtype, H, heads, kvh, Fh = torch.bfloat16, 256, 4, 2, 512
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
        dtype, H, heads, kvh, Fh = torch.float32, 64, 4, 2, 96
    cfg = TransformerConfig(vocab_size=200, hidden_size=H, num_layers=2, num_heads=heads, num_kv_heads=kvh, ffn_hidden_size=Fh,
                            max_seq_len=256, init_std=0.08)
    model = DenseModel(cfg, device=dev, dtype=dtype, seed=4)
    greedy = SamplerConfig(temperature=0.0, top_k=0, top_p=1.0)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(3, 200, (n,), generator=g).tolist() for n in (5, 40, 17)]
    eng = TPInferenceEngine(model, None, EngineConfig(max_batch=8, num_pages=64), rank, world, symm)
    outs = eng.generate_batch(prompts, max_tokens=8, sampling=greedy)
    res = {"outs": outs, "allreduce_calls": eng.allreduce_calls, "local_heads": eng.model.cfg.num_heads,
           "kv_bytes_per_token": eng.cache.bytes_per_token()}
    if rank == 0:
        ref = InferenceEngine(model, None, EngineConfig(max_batch=8, num_pages=64, cuda_graph=False))
        res["ref"] = ref.generate_batch(prompts, max_tokens=8, sampling=greedy)
        res["ref_kv_bytes_per_token"] = ref.cache.bytes_per_token()
    if where == "cuda":
        from transformers_fusion_b200.ops import _lib
        torch.cuda.synchronize()
        res["status"] = int(_lib.status_word(dev)[0].item())
    json.dump(res, open(os.path.join(out_dir, f"rank{rank}.json"), "w"))
    dist.barrier()
    if symm is not None:
        symm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
