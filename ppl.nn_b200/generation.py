"""Step driver: the ragged index tensors of every step of a batch of generation requests, with the same
semantics as ppl.nn's benchmark driver (tools/benchmark_llama/generation_state.cc:5-192):

  * ``prepare``     per request: cache capacity = prompt length + generation length - 1 tokens (rounded up to
                    whole pages in paged mode); totals and the number of steps (:5-58);
  * ``first_step``  every request as a prefill sequence: seq_lengths = kv_lengths = prompt length,
                    start_pos 0, decoding_batches 0, cache regions handed out back to back (or page by
                    page) in request order (:60-123);
  * ``next_step``   requests that have produced all their tokens leave the batch, the others are compacted
                    to the front (their cache regions travel with them) and become decode sequences:
                    start_pos = previous kv length, kv length + 1, seq length 1,
                    decoding_batches = batch size (:125-192).

The driver only builds indices; the caller runs the model (here: one attention layer) between steps.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


@dataclass
class Request:
    prompt_len: int
    generation_len: int


@dataclass
class ModelIO:
    """What one step feeds to the operators (int64 numpy arrays; host scalars as ints)."""
    seq_starts: np.ndarray
    kv_starts: np.ndarray
    start_pos: np.ndarray
    cache_indices: np.ndarray  # [batch] token rows, or [batch, max_cache_pages] first rows of pages
    decoding_batches: int
    max_seq_len: int
    max_kv_len: int
    batch_slots: np.ndarray    # request index of every sequence of the step

    @property
    def batch(self) -> int:
        return int(self.start_pos.shape[0])

    @property
    def seq_lengths(self) -> np.ndarray:
        return np.diff(self.seq_starts)

    @property
    def kv_lengths(self) -> np.ndarray:
        return np.diff(self.kv_starts)


class GenerationState:
    def __init__(self, cache_mode: int = 0, page_size: int = 128):
        if cache_mode not in (0, 1):
            raise ValueError(f"unknown cache_mode: {cache_mode}")
        self.cache_mode = cache_mode
        self.page_size = page_size
        self.requests: list[Request] = []
        self.current_step = -1

    # generation_state.cc:5-58
    def prepare(self, requests: list[Request]) -> None:
        for r in requests:
            if r.generation_len <= 0:
                raise ValueError("generation_len of request must not be 0")
        self.requests = list(requests)
        self.total_batch_size = len(requests)
        self.total_input_length = sum(r.prompt_len for r in requests)
        self.total_output_length = sum(r.generation_len for r in requests)
        self.max_steps = max((r.generation_len for r in requests), default=0)
        cache_len = [r.prompt_len + r.generation_len - 1 for r in requests]
        if self.cache_mode == 0:
            self.total_cache_length = sum(cache_len)
            self.total_cache_pages = 0
            self.max_cache_pages = 0
        else:
            pages = [(c + self.page_size - 1) // self.page_size for c in cache_len]
            self.total_cache_pages = sum(pages)
            self.max_cache_pages = max(pages, default=0)
            self.total_cache_length = self.total_cache_pages * self.page_size
        self.current_step = -1

    # generation_state.cc:60-123
    def first_step(self) -> ModelIO:
        n = self.total_batch_size
        self.current_step = 0
        self.current_batch_size = n
        seq = np.array([r.prompt_len for r in self.requests], dtype=np.int64)
        self._kv_lengths = seq.copy()
        self._slots = np.arange(n, dtype=np.int64)
        if self.cache_mode == 0:
            cap = np.array([r.prompt_len + r.generation_len - 1 for r in self.requests], dtype=np.int64)
            self._cache = np.concatenate([[0], np.cumsum(cap)[:-1]]).astype(np.int64) if n else np.zeros(0, np.int64)
        else:
            self._cache = np.zeros((n, max(self.max_cache_pages, 1)), dtype=np.int64)
            row = 0
            for i, r in enumerate(self.requests):
                pages = (r.prompt_len + r.generation_len - 1 + self.page_size - 1) // self.page_size
                for p in range(pages):
                    self._cache[i, p] = row
                    row += self.page_size
        self._max_kv_len = int(seq.max()) if n else 0
        return ModelIO(seq_starts=np.concatenate([[0], np.cumsum(seq)]).astype(np.int64),
                       kv_starts=np.concatenate([[0], np.cumsum(seq)]).astype(np.int64),
                       start_pos=np.zeros(n, dtype=np.int64), cache_indices=self._cache.copy(), decoding_batches=0,
                       max_seq_len=self._max_kv_len, max_kv_len=self._max_kv_len, batch_slots=self._slots.copy())

    # generation_state.cc:125-192
    def next_step(self) -> ModelIO | None:
        if self.current_step < 0:
            raise RuntimeError("first_step() comes first")
        done = np.array([self.current_step + 1 >= self.requests[s].generation_len for s in self._slots], dtype=bool)
        if self.current_step + 1 >= self.max_steps:
            return None
        self.current_step += 1
        keep = ~done
        start_pos = self._kv_lengths[keep]
        self._kv_lengths = start_pos + 1
        self._slots = self._slots[keep]
        self._cache = self._cache[keep]
        self.current_batch_size = int(keep.sum())
        n = self.current_batch_size
        self._max_kv_len = max(self._max_kv_len, int(self._kv_lengths.max()) if n else 0)  # never shrinks (:158)
        return ModelIO(seq_starts=np.arange(n + 1, dtype=np.int64),
                       kv_starts=np.concatenate([[0], np.cumsum(self._kv_lengths)]).astype(np.int64),
                       start_pos=start_pos.astype(np.int64), cache_indices=self._cache.copy(), decoding_batches=n,
                       max_seq_len=1, max_kv_len=self._max_kv_len, batch_slots=self._slots.copy())

    def steps(self):
        """All steps of the batch, first to last."""
        io = self.first_step()
        while io is not None:
            yield io
            io = self.next_step()
