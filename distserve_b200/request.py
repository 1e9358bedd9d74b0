"""The request-side data carriers of the migration path
(distserve/request.py: Request 172-296, MigratingRequest 408-433), reduced to
what block accounting reads: ids and token counts.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List

from .config import ParallelConfig


@dataclass
class Request:
    request_id: int
    prompt_token_ids: List[int]
    generated_token_ids: List[int] = field(default_factory=list)
    generated_tokens: List[str] = field(default_factory=list)

    @classmethod
    def of_length(cls, request_id: int, prompt_len: int) -> "Request":
        return cls(request_id, [0] * prompt_len)

    def get_input_len(self) -> int:
        return len(self.prompt_token_ids)

    def get_output_len(self) -> int:
        if len(self.generated_tokens) != len(self.generated_token_ids):
            raise AssertionError("generated_tokens and generated_token_ids are out of step")
        return len(self.generated_token_ids)

    def append_token(self, token_id: int = 0, token: str = "") -> None:
        self.generated_token_ids.append(token_id)
        self.generated_tokens.append(token)


@dataclass
class MigratingRequest:
    """A request that finished prefill and whose blocks still sit in the
    context stage's pools (an element of the bridge queue)."""

    req: Request
    block_indexes: List[int]
    context_parallel_config: ParallelConfig
