"""Per-request state: tokens, block table, scheduling counters (reference: engine/sequence.py:11-112)."""
from __future__ import annotations

import time
from enum import Enum, auto
from itertools import count

from .sampling_params import SamplingParams


class SequenceStatus(Enum):
    WAITING = auto()
    RUNNING = auto()
    SWAPPED = auto()
    FINISHED = auto()


class Sequence:
    block_size: int = 16
    _counter = count()

    def __init__(self, token_ids: list, sampling_params: SamplingParams | None = None):
        if len(token_ids) == 0:
            raise ValueError("Prompt must contain at least one token")
        sp = sampling_params or SamplingParams()
        self.seq_id = next(Sequence._counter)
        self.status = SequenceStatus.WAITING
        self.token_ids = list(token_ids)
        self.last_token = token_ids[-1]
        self.num_tokens = len(self.token_ids)
        self.num_prompt_tokens = len(token_ids)
        self.num_cached_tokens = 0          # tokens whose KV / recurrent state is in the cache
        self.num_scheduled_tokens = 0       # tokens to run this step
        self.is_prefill = True
        self.block_table: list = []
        self.cpu_block_table: list = []     # host blocks while SWAPPED
        self.sampling_params = sp
        self.temperature = sp.temperature
        self.max_tokens = sp.max_tokens
        self.ignore_eos = sp.ignore_eos
        self.top_p = sp.top_p
        self.top_k = sp.top_k
        self.repetition_penalty = sp.repetition_penalty
        self.stop = sp.stop
        self.deltanet_state_slot = -1
        self.constraint = None
        self.constraint_state = None
        self.prefix_restore_key = None      # prefix-cache node whose DeltaNet snapshot must be restored
        self.snapshot_points: list = []     # absolute token counts at which to snapshot DeltaNet state
        self.finish_reason = None           # "stop" | "length"
        self.arrival_time = time.perf_counter()
        self.first_token_time = None
        self.token_times: list = []
        self.num_preemptions = 0

    def __len__(self):
        return self.num_tokens

    def __getitem__(self, key):
        return self.token_ids[key]

    @property
    def is_finished(self):
        return self.status == SequenceStatus.FINISHED

    @property
    def num_completion_tokens(self):
        return self.num_tokens - self.num_prompt_tokens

    @property
    def prompt_token_ids(self):
        return self.token_ids[:self.num_prompt_tokens]

    @property
    def completion_token_ids(self):
        return self.token_ids[self.num_prompt_tokens:]

    @property
    def num_blocks(self):
        return (self.num_tokens + self.block_size - 1) // self.block_size

    @property
    def last_block_num_tokens(self):
        return self.num_tokens - (self.num_blocks - 1) * self.block_size

    def block(self, i):
        assert 0 <= i < self.num_blocks
        return self.token_ids[i * self.block_size:(i + 1) * self.block_size]

    def append_token(self, token_id: int):
        self.token_ids.append(token_id)
        self.last_token = token_id
        self.num_tokens += 1

    _STATE = ("seq_id", "status", "num_tokens", "num_prompt_tokens", "num_cached_tokens",
              "num_scheduled_tokens", "block_table", "token_ids", "last_token", "is_prefill",
              "temperature", "max_tokens", "ignore_eos", "top_p", "top_k", "deltanet_state_slot",
              "repetition_penalty", "stop", "sampling_params", "finish_reason")

    def __getstate__(self):
        return tuple(getattr(self, k) for k in self._STATE)

    def __setstate__(self, state):
        for k, v in zip(self._STATE, state):
            setattr(self, k, v)
        self.cpu_block_table, self.constraint, self.constraint_state = [], None, None
        self.prefix_restore_key, self.snapshot_points = None, []
        self.arrival_time, self.first_token_time, self.token_times, self.num_preemptions = 0.0, None, [], 0
