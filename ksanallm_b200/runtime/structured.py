"""Per-request cursor over the structured-output state machine. After every sampled token the
generated text is checked: constant segments are injected (and the whole generated text is
re-tokenised, which fixes token boundaries), free segments end when the next constant begins, the
final state finishes the request (src/ksana_llm/batch_scheduler/strategy/continuous_batching.cpp:57-138).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List


@dataclass
class StructuredAction:
    changed: bool
    final: bool
    tokens: List[int]


class StructuredOutput:
    def __init__(self, fsm, tokenizer):
        if tokenizer is None:
            raise ValueError("structured output needs a tokenizer")
        self.fsm, self.tokenizer = fsm, tokenizer
        self.segment, self.segment_start = 0, 0

    def initial_tokens(self) -> List[int]:
        """Constant text the pattern starts with (injected before the first sampled token)."""
        changed, final, text, seg, start = self.fsm.step("", 0, 0)
        self.segment, self.segment_start = seg, start
        return self.tokenizer.encode(text, add_special_tokens=False) if text else []

    def after_token(self, generated: List[int]) -> StructuredAction:
        text = self.tokenizer.decode(generated, skip_special_tokens=True)
        changed, final, new_text, seg, start = self.fsm.step(text, self.segment, self.segment_start)
        self.segment, self.segment_start = seg, start
        if changed or final:
            toks = self.tokenizer.encode(new_text, add_special_tokens=False) if changed else list(generated)
            return StructuredAction(changed, final, list(toks))
        return StructuredAction(False, False, list(generated))
