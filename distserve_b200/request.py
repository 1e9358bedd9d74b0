"""The request-side data carriers of the migration path
(distserve/request.py: Request 172-296, MigratingRequest 408-433), reduced to
what block accounting reads: ids and token counts.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

from .config import ParallelConfig


@dataclass
class Request:
    request_id: int
    prompt_token_ids: List[int]
    generated_token_ids: List[int] = field(default_factory=list)
    generated_tokens: List[str] = field(default_factory=list)
    max_tokens: int = 16          # SamplingParams.max_tokens of the reference (distserve/request.py:49-83)
    is_finished: bool = False

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

    def add_generated_token(self, token: str = "", token_id: int = 0) -> None:
        """One decoding step's result; the request finishes when it has produced max_tokens tokens
        (distserve/request.py:205-222, stop strings aside)."""
        self.append_token(token_id, token)
        if self.get_output_len() >= self.max_tokens:
            self.is_finished = True

    def is_context_stage(self) -> bool:
        return len(self.generated_tokens) == 0

    def get_num_input_tokens(self) -> int:
        """Tokens the next iteration feeds: the whole prompt before the first token exists, one afterwards."""
        return len(self.prompt_token_ids) if self.is_context_stage() else 1


class BatchedRequests:
    """The requests of one iteration (distserve/request.py:297-372, the parts the schedulers use)."""

    def __init__(self, requests: Optional[List[Request]] = None) -> None:
        self.requests: List[Request] = [] if requests is None else requests

    def __len__(self) -> int:
        return len(self.requests)

    def add_request(self, request: Request) -> None:
        assert request.request_id not in self.get_request_ids(), f"request {request.request_id} already exists"
        self.requests.append(request)

    def pop_finished_requests(self) -> List[Request]:
        finished = [r for r in self.requests if r.is_finished]
        self.requests = [r for r in self.requests if not r.is_finished]
        return finished

    def get_request_ids(self) -> List[int]:
        return [r.request_id for r in self.requests]

    def get_num_input_tokens(self) -> int:
        return sum(r.get_num_input_tokens() for r in self.requests)


@dataclass
class MigratingRequest:
    """A request that finished prefill and whose blocks still sit in the
    context stage's pools (an element of the bridge queue)."""

    req: Request
    block_indexes: List[int]
    context_parallel_config: ParallelConfig
