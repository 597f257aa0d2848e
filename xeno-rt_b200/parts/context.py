"""What a step hands to every part: the tokens of the step as flat device arrays."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..core import DType


@dataclass
class StepContext:
    """The tokens of one step, all sequences laid end to end (T tokens of n sequences).

    Device tensors (int32): ``token_ids`` [T]; ``tok_pos`` [T] absolute position of each token in
    its sequence; ``tok_slot`` [T] cache slot of each token (-1 marks a padding row, which every
    kernel skips); ``cu_seqlens`` [n + 1] where each sequence's tokens begin; ``seq_slot`` [n];
    ``seq_start`` [n] length of each sequence before this step.
    Host values: ``new_lens`` tokens each sequence brings; ``starts``; ``all_single`` every
    sequence brings exactly one token (a decode step); ``max_new`` and ``max_context`` the
    largest new-token count and the largest length after the step; ``mean_context`` the lengths
    after the step summed over the sequences and divided by the rows of the step (0: not known).
    ``shared`` holds what parts compute once per step and share across layers (rotation tables).
    """
    n_tokens: int
    n_seqs: int
    token_ids: torch.Tensor
    tok_pos: torch.Tensor
    tok_slot: torch.Tensor
    cu_seqlens: torch.Tensor
    seq_slot: torch.Tensor
    seq_start: torch.Tensor
    new_lens: list
    starts: list
    all_single: bool
    max_new: int
    max_context: int
    dtype: DType
    mean_context: int = 0
    captured: bool = False  # the step is being captured into (or replayed from) a CUDA graph:
    #                         launch shapes must not depend on the sequences' lengths
    shared: dict = field(default_factory=dict)
    # A part that adds into the residual stream may prepare the norm that follows it: the arrangement
    # names that norm in ``then_norm`` before it calls the part, and a part that did so leaves the
    # result (a parts.norm.PendingNorm) in ``pending``.  Parts that know nothing of this leave both alone.
    then_norm: object = None
    pending: object = None

    def take_pending(self, norm):
        """The prepared result of ``norm`` if the part that ran last left one, else None."""
        pending, self.pending, self.then_norm = self.pending, None, None
        return pending if pending is not None and pending.norm is norm else None


def context_bucket(max_context: int) -> int:
    """The power of two (at least 256) at or above a context length.  Launch shapes that depend on
    the context (how attention splits the keys) are chosen from this, so that they change only
    when a power of two is crossed: a captured CUDA graph stays valid in between, and a step gives
    the same result replayed from a graph or launched kernel by kernel."""
    return max(256, 1 << (max(1, int(max_context)) - 1).bit_length())
