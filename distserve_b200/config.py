"""Shard geometry of the two stages: the part of ``distserve/config.py`` the
KV-migration path depends on, with the same attribute and method names so the
worker and block-manager mirrors read like their reference counterparts.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple

GB = 1 << 30


class ParallelConfig:
    """Position of one worker in its stage (distserve/config.py:32-66)."""

    def __init__(self, tensor_parallel_size: int = 1, tensor_parallel_rank: int = 0,
                 pipeline_parallel_size: int = 1, pipeline_parallel_rank: int = 0) -> None:
        if tensor_parallel_size < 1 or pipeline_parallel_size < 1:
            raise ValueError("parallel sizes must be >= 1")
        if not (0 <= tensor_parallel_rank < tensor_parallel_size and 0 <= pipeline_parallel_rank < pipeline_parallel_size):
            raise ValueError("parallel rank out of range")
        self.tensor_parallel_size = tensor_parallel_size
        self.tensor_parallel_rank = tensor_parallel_rank
        self.pipeline_parallel_size = pipeline_parallel_size
        self.pipeline_parallel_rank = pipeline_parallel_rank
        self.world_size = tensor_parallel_size * pipeline_parallel_size
        self.use_parallel = self.world_size > 1

    def to_list(self) -> List[int]:
        """[tp_size, tp_rank, pp_size, pp_rank] — the order the native
        register call expects (distserve/config.py:57-63)."""
        return [self.tensor_parallel_size, self.tensor_parallel_rank,
                self.pipeline_parallel_size, self.pipeline_parallel_rank]

    def with_rank(self, pp_rank: int, tp_rank: int) -> "ParallelConfig":
        return ParallelConfig(self.tensor_parallel_size, tp_rank, self.pipeline_parallel_size, pp_rank)

    def is_last_stage(self) -> bool:
        return self.pipeline_parallel_rank == self.pipeline_parallel_size - 1

    def __repr__(self) -> str:
        return (f"ParallelConfig(tp={self.tensor_parallel_size}, tp_rank={self.tensor_parallel_rank}, "
                f"pp={self.pipeline_parallel_size}, pp_rank={self.pipeline_parallel_rank})")


class CacheConfig:
    """Block size and per-request block cap (distserve/config.py CacheConfig)."""

    def __init__(self, block_size: int, max_num_blocks_per_req: int,
                 gpu_memory_utilization: float = 0.9, cpu_swap_space: int = 0) -> None:
        self.block_size = block_size
        self.max_num_blocks_per_req = max_num_blocks_per_req
        self.gpu_memory_utilization = gpu_memory_utilization
        self.cpu_swap_space = cpu_swap_space * GB


@dataclass(frozen=True)
class KVModelConfig:
    """The model facts the KV pools depend on.  The reference reads them from a
    HuggingFace config (distserve/config.py:225-257,279-286); this path needs
    only the counts, so they are given directly."""

    num_layers: int          # global transformer layers
    num_kv_heads: int        # global KV heads (== attention heads unless GQA/MQA)
    head_dim: int
    dtype: str = "float16"   # "float16" | "bfloat16" | "float32"

    def get_num_layers(self, parallel_config: ParallelConfig = ParallelConfig()) -> int:
        pp = parallel_config.pipeline_parallel_size
        if self.num_layers % pp:
            raise ValueError(f"{self.num_layers} layers do not split over {pp} pipeline stages")
        return self.num_layers // pp

    def get_num_heads(self, parallel_config: ParallelConfig = ParallelConfig()) -> int:
        tp = parallel_config.tensor_parallel_size
        if self.num_kv_heads == 1:
            return 1      # multi-query attention: every rank holds the one KV head (distserve/config.py:233-237)
        if self.num_kv_heads % tp:
            raise ValueError(f"{self.num_kv_heads} KV heads do not split over {tp} tensor-parallel ranks")
        return self.num_kv_heads // tp

    def get_head_size(self) -> int:
        return self.head_dim

    def get_dtype_size(self) -> int:
        return {"float16": 2, "bfloat16": 2, "float32": 4}[self.dtype]

    def get_torch_dtype(self):
        import torch

        return {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}[self.dtype]

    def layer_range(self, pc: ParallelConfig) -> Tuple[int, int]:
        """Global layers held by a worker: pipeline rank i holds the i-th run."""
        n = self.get_num_layers(pc)
        return pc.pipeline_parallel_rank * n, (pc.pipeline_parallel_rank + 1) * n

    def head_range(self, pc: ParallelConfig) -> Tuple[int, int]:
        """Global KV heads held by a worker: tensor rank i holds the i-th chunk."""
        n = self.get_num_heads(pc)
        if self.num_kv_heads == 1:
            return 0, 1
        return pc.tensor_parallel_rank * n, (pc.tensor_parallel_rank + 1) * n

    def block_bytes(self, pc: ParallelConfig, block_size: int) -> int:
        """Bytes of one block of one pool (K or V) on a worker."""
        return self.get_num_layers(pc) * self.get_num_heads(pc) * block_size * self.head_dim * self.get_dtype_size()


@dataclass(frozen=True)
class Overlap:
    """One context worker's contribution to one decoding worker's rectangle."""

    ctx_pp_rank: int
    ctx_tp_rank: int
    src_layers: Tuple[int, int]   # local layer range inside the context worker's pool
    src_heads: Tuple[int, int]
    dst_layers: Tuple[int, int]   # local layer range inside the decoding worker's pool
    dst_heads: Tuple[int, int]


def plan_overlaps(model: KVModelConfig, ctx: ParallelConfig, dec: ParallelConfig) -> List[Overlap]:
    """Context workers that a decoding worker pulls from, by interval
    intersection of the layer and head ranges.  `ctx` supplies only the stage's
    sizes; `dec` names one decoding worker."""
    dl0, dl1 = model.layer_range(dec)
    dh0, dh1 = model.head_range(dec)
    out: List[Overlap] = []
    # With a single KV head every context rank holds it; a decoding rank reads the replica at the matching position.
    replica = dec.tensor_parallel_rank * ctx.tensor_parallel_size // dec.tensor_parallel_size
    for p in range(ctx.pipeline_parallel_size):
        for t in range(ctx.tensor_parallel_size):
            if model.num_kv_heads == 1 and t != replica:
                continue
            c = ctx.with_rank(p, t)
            cl0, cl1 = model.layer_range(c)
            ch0, ch1 = model.head_range(c)
            l0, l1, h0, h1 = max(dl0, cl0), min(dl1, cl1), max(dh0, ch0), min(dh1, ch1)
            if l0 < l1 and h0 < h1:
                out.append(Overlap(p, t, (l0 - cl0, l1 - cl0), (h0 - ch0, h1 - ch0),
                                   (l0 - dl0, l1 - dl0), (h0 - dh0, h1 - dh0)))
    return out
