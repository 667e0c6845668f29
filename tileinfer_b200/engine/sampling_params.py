"""Per-request sampling and constrained-decoding parameters.

Field names and defaults are those of the reference (engine/sampling_params.py:5-31) so callers
can switch without edits.  `n` is accepted and, as in the reference, only n == 1 is generated.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field


@dataclass
class SamplingParams:
    temperature: float = 0.6
    top_p: float = 1.0
    top_k: int = -1
    max_tokens: int = 256
    ignore_eos: bool = False
    repetition_penalty: float = 1.0
    stop: list = field(default_factory=list)
    n: int = 1
    logit_bias: dict = field(default_factory=dict)
    allowed_token_ids: list = field(default_factory=list)
    bad_token_ids: list = field(default_factory=list)
    guided_choice: list = field(default_factory=list)
    guided_json: object = None
    guided_regex: str = None
    seed: int = None

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.repetition_penalty < 1.0:
            raise ValueError(f"repetition_penalty must be >= 1.0, got {self.repetition_penalty}")
        if self.max_tokens <= 0:
            raise ValueError(f"max_tokens must be > 0, got {self.max_tokens}")
        if self.top_k == 0 or self.top_k < -1:
            raise ValueError(f"top_k must be -1 (off) or >= 1, got {self.top_k}")
        if isinstance(self.stop, str):
            self.stop = [self.stop]
        self.logit_bias = {int(k): float(v) for k, v in (self.logit_bias or {}).items()}

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0 or self.top_k == 1

    @property
    def has_constraint(self) -> bool:
        return bool(self.logit_bias or self.allowed_token_ids or self.bad_token_ids
                    or self.guided_choice or self.guided_json or self.guided_regex)

    # Full serialisation: the server sends every field to the tensor-parallel workers, so that
    # stop strings and guided decoding cannot desynchronise the ranks.
    def to_json(self) -> str:
        return json.dumps(asdict(self))

    @classmethod
    def from_json(cls, s: str) -> "SamplingParams":
        return cls(**json.loads(s))
