"""Sharded checkpoints for ZeRO / FSDP runs: every rank writes only what it owns, a manifest ties the pieces together.

  <dir>/manifest.json            {"world", "numel", "padded", "step", "dtype", "shards": [{"rank", "lo", "hi", "file"}], ...}
  <dir>/model.rank{r}.shard      raw little-endian fp32: this rank's slice [lo, hi) of the flat master parameters,
                                 followed by the optimiser moments of the same slice (m then v) when present

Loading with the same world reads one file per rank; loading with a different world re-cuts the slices (each new rank
reads the byte ranges of the old files that overlap its slice), so a job can resume on more or fewer GPUs.
``consolidate`` rebuilds the single-file ``.quant`` checkpoint from the shards.

Reference counterparts: FSDP::save_sharded_checkpoint / load_sharded_checkpoint (``model.rank{r}.quant`` + manifest,
src/trainer/fsdp.cpp:560-640) and ZeroOptimizer::save_state / load_state (zero_optimizer_core.cpp)."""
from __future__ import annotations

import json
import os
from typing import Optional, Tuple

import numpy as np
import torch


def _shard_path(d: str, rank: int) -> str:
    return os.path.join(d, f"model.rank{rank}.shard")


def save_shard(d: str, rank: int, world: int, numel: int, lo: int, hi: int, master: torch.Tensor, m: Optional[torch.Tensor] = None,
               v: Optional[torch.Tensor] = None, step: int = 0, extra: Optional[dict] = None) -> None:
    """Writes this rank's slice.  ``master`` / ``m`` / ``v`` are the [hi - lo] fp32 slices.  Rank 0 also writes the manifest
    (slices are the equal cuts of a buffer padded to ``world`` equal parts, so rank 0 can describe all of them)."""
    os.makedirs(d, exist_ok=True)
    assert master.numel() == hi - lo
    with open(_shard_path(d, rank), "wb") as f:
        f.write(master.detach().float().cpu().numpy().tobytes())
        if m is not None:
            f.write(m.detach().float().cpu().numpy().tobytes())
            f.write((v if v is not None else torch.zeros_like(m)).detach().float().cpu().numpy().tobytes())
    if rank == 0:
        per = hi - lo
        man = {"world": world, "numel": numel, "padded": per * world, "step": step, "has_moments": m is not None,
               "shards": [{"rank": r, "lo": r * per, "hi": (r + 1) * per, "file": os.path.basename(_shard_path(d, r))} for r in range(world)]}
        man.update(extra or {})
        with open(os.path.join(d, "manifest.json"), "w") as f:
            json.dump(man, f, indent=1)


def read_manifest(d: str) -> dict:
    with open(os.path.join(d, "manifest.json")) as f:
        return json.load(f)


def _read_range(d: str, man: dict, lo: int, hi: int, part: int) -> torch.Tensor:
    """Elements [lo, hi) of section ``part`` (0 master, 1 m, 2 v) gathered from the old shard files."""
    out = np.zeros(hi - lo, dtype=np.float32)
    for sh in man["shards"]:
        a, b = max(lo, sh["lo"]), min(hi, sh["hi"])
        if a >= b:
            continue
        per = sh["hi"] - sh["lo"]
        with open(os.path.join(d, sh["file"]), "rb") as f:
            f.seek(4 * (part * per + a - sh["lo"]))
            out[a - lo:b - lo] = np.frombuffer(f.read(4 * (b - a)), dtype=np.float32)
    return torch.from_numpy(out)


def load_shard(d: str, rank: int, world: int) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor], dict]:
    """This rank's slice under a (possibly different) world size: (master, m, v, manifest).  The flat length is re-padded
    to ``world`` equal parts; elements past the old padded length read as zero."""
    man = read_manifest(d)
    n = man["numel"]
    per = -(-max(n, 1) // world)
    per = -(-per // 1024) * 1024 if man["padded"] % 1024 == 0 else per
    lo, hi = rank * per, (rank + 1) * per
    master = _read_range(d, man, lo, hi, 0)
    m = v = None
    if man.get("has_moments"):
        m, v = _read_range(d, man, lo, hi, 1), _read_range(d, man, lo, hi, 2)
    return master, m, v, man


def consolidate(d: str) -> torch.Tensor:
    """The whole flat fp32 parameter vector (without padding)."""
    man = read_manifest(d)
    return _read_range(d, man, 0, man["numel"], 0)


def save_engine(engine, d: str, step: int = 0) -> None:
    """Sharded save of a TrainEngine (ZeRO stage >= 1: each rank its slice; stage 0: rank 0 writes one whole 'shard')."""
    flat, opt = engine.flat, engine.opt
    lo, hi = engine.shard
    world, rank = (engine.world, engine.rank) if engine.zero_stage >= 1 else (1, 0)
    if engine.zero_stage == 0 and engine.rank != 0:
        return
    master = getattr(opt, "master", None)
    master = master if master is not None else flat.params[lo:hi].float()
    save_shard(d, rank, world, flat.numel, lo, hi, master, getattr(opt, "m", None), getattr(opt, "v", None), step,
               {"opt_step": int(getattr(opt, "step_count", step))})


def load_engine(engine, d: str) -> int:
    """Restores a TrainEngine from a sharded checkpoint written under any world size.  Returns the saved step."""
    flat, opt = engine.flat, engine.opt
    lo, hi = engine.shard
    man = read_manifest(d)
    master = _read_range(d, man, lo, hi, 0).to(flat.params.device)
    if getattr(opt, "master", None) is not None:
        opt.master.copy_(master)
    flat.params[lo:hi].copy_(master.to(flat.params.dtype))
    if man.get("has_moments") and getattr(opt, "m", None) is not None:
        opt.m.copy_(_read_range(d, man, lo, hi, 1).to(opt.m.device))
        opt.v.copy_(_read_range(d, man, lo, hi, 2).to(opt.v.device))
    if hasattr(opt, "step_count"):
        opt.step_count = int(man.get("opt_step", man.get("step", 0)))
    if engine.world > 1 and engine.zero_stage >= 1:
        import torch.distributed as dist
        dist.all_gather_into_tensor(flat.params, flat.params[lo:hi].clone(), group=engine.group)
    elif engine.zero_stage == 0:
        full = _read_range(d, man, 0, flat.numel, 0).to(flat.params.device)
        flat.params.copy_(full.to(flat.params.dtype))
    return int(man.get("step", 0))
