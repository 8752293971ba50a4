"""Sampling options of a request, with the reference's names and meanings
(crates/sglang-srt/src/types.rs:16-37; validation ranges of the request layer,
crates/sglang-srt/src/router.rs:31-71).  ``seed`` is an addition: the reference draws from
the thread's generator and has no seed option (crates/sglang-srt/src/model_executor.rs:392-403).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

GREEDY_EPSILON = 1.1920929e-07       # f32::EPSILON: a temperature at or below it is greedy


@dataclass(frozen=True)
class SamplingParams:
    max_new_tokens: int = 128
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    min_p: Optional[float] = None
    frequency_penalty: Optional[float] = None
    presence_penalty: Optional[float] = None
    repetition_penalty: Optional[float] = None
    stop_token_ids: Tuple[int, ...] = ()
    ignore_eos: bool = False
    seed: Optional[int] = None

    def __post_init__(self):
        def bad(message):
            raise ValueError(f"sampling_params: {message}")
        if self.max_new_tokens < 0:
            bad("max_new_tokens must be non-negative")
        if self.temperature is not None and not self.temperature >= 0.0:
            bad("temperature must be non-negative")
        if self.top_p is not None and not 0.0 < self.top_p <= 1.0:
            bad("top_p must be in (0, 1]")
        if self.min_p is not None and not 0.0 <= self.min_p <= 1.0:
            bad("min_p must be in [0, 1]")
        for name in ("frequency_penalty", "presence_penalty"):
            value = getattr(self, name)
            if value is not None and not -2.0 <= value <= 2.0:
                bad(f"{name} must be in [-2, 2]")
        if self.repetition_penalty is not None and not 0.0 < self.repetition_penalty <= 2.0:
            bad("repetition_penalty must be in (0, 2]")

    @classmethod
    def from_dict(cls, options: Optional[Mapping[str, Any]]) -> "SamplingParams":
        options = dict(options or {})
        for key in ("n", "best_of"):
            if options.pop(key, 1) not in (1, None):
                raise ValueError(f"sampling_params: {key} must be 1")
        stops = list(options.pop("stop_token_ids", None) or [])
        single = options.pop("stop_token_id", None)
        if single is not None:
            stops.append(single)
        unknown = set(options) - set(cls.__dataclass_fields__)
        if unknown:
            raise ValueError(f"sampling_params: unknown options {sorted(unknown)}")
        return cls(stop_token_ids=tuple(int(s) for s in stops), **options)

    # -- the reference's decision of how a row is sampled (model_executor.rs:458-469)
    @property
    def is_greedy(self) -> bool:
        if self.temperature is None and self.top_p is None and self.top_k is None and self.min_p is None:
            return True
        return self.effective_temperature <= GREEDY_EPSILON or self.top_k == 1

    @property
    def effective_temperature(self) -> float:
        return 1.0 if self.temperature is None else float(self.temperature)

    @property
    def filters(self) -> bool:
        """True if the candidates are cut by top-k, top-p or min-p."""
        return (self.top_k is not None and self.top_k > 0) or (self.top_p is not None and self.top_p < 1.0) \
            or (self.min_p is not None and self.min_p > 0.0)

    @property
    def has_penalties(self) -> bool:
        return (self.frequency_penalty or 0.0) != 0.0 or (self.presence_penalty or 0.0) != 0.0 \
            or (self.repetition_penalty if self.repetition_penalty is not None else 1.0) != 1.0
