"""A decode loop that carries one paged cache across steps and layers.

The reference threads a single dense cache object through all blocks of a forward pass and
reassigns it per block (src/core/transformer.py:229-238), so block ``i+1`` attends over block
``i``'s keys, and its ``generate`` re-runs the whole sequence on every step with a cache that was
built empty before the loop and is never fed back (transformer.py:273-290).  ``decode_loop`` is
the corrected form for attention layers of this package: every layer owns one pool of a shared
``PagedKVCache`` (``cache.layer(i)``: one allocator, one block table, one upload of the step's
bookkeeping), the prompt is appended once, and each later step appends one token per sequence
and attends over the pages already in place.
"""

from __future__ import annotations

from typing import Callable, Iterable, List, Optional, Sequence, Union

import torch

__all__ = ["decode_loop"]


@torch.no_grad()
def decode_loop(layers: Sequence, cache, x_steps: Union[Iterable[torch.Tensor], Callable], *,
                residual: bool = True, sliding_window: Optional[int] = None, sink_cfg: Optional[dict] = None,
                max_steps: Optional[int] = None) -> List[torch.Tensor]:
    """Run inputs through ``layers`` (attention modules with the reference's ``forward`` signature,
    e.g. ``AttentionB200``) step by step; layer ``i`` reads and extends ``cache.layer(i)``.

    ``x_steps`` is either an iterable of ``[B,S,d_model]`` tensors -- typically the prompt
    (``S`` tokens) followed by single-token steps -- or a callable ``next_x(prev_out, t)`` that
    receives the previous step's output (``None`` for ``t = 0``) and returns the next input, or
    ``None`` to stop; that is the autoregressive form, where step ``t+1`` is built from step ``t``.
    ``residual=True`` adds each layer's output to its input (the residual stream of
    src/core/transformer.py:125-132 without the feed-forward half).  Returns the per-step outputs
    of the last layer.
    """
    if cache.n_layers != len(layers):
        raise ValueError(f"{len(layers)} layers but the cache holds {cache.n_layers}")
    views = [cache.layer(i) for i in range(len(layers))]
    outs: List[torch.Tensor] = []

    def one(x: torch.Tensor) -> torch.Tensor:
        h = x
        for layer, view in zip(layers, views):
            y, _ = layer(h, kv_cache=view, sliding_window=sliding_window,
                         sink_cfg=sink_cfg if (sink_cfg is not None and x.shape[1] == 1) else None)
            h = h + y if residual else y
        return h

    if callable(x_steps):
        prev, t = None, 0
        while max_steps is None or t < max_steps:
            x = x_steps(prev, t)
            if x is None:
                break
            prev = one(x)
            outs.append(prev)
            t += 1
    else:
        for t, x in enumerate(x_steps):
            if max_steps is not None and t >= max_steps:
                break
            outs.append(one(x))
    return outs
