"""Block arrangements: how norms, mixer, feed-forward and the residual stream
are put together.

``sandwich`` (norm before and after each sub-layer; the post norm comes
before the add, as in src/model/layer.rs:1101-1192):

    h += post_mixer(mixer(pre_mixer(h)))
    h += post_feed_forward(feed_forward(pre_feed_forward(h)))

``pre_norm`` is the same arrangement without the two post norms.  The
residual stream h is kept and summed in 32-bit.  When the norms around an
add are RMS norms the block runs "norm of the sub-layer's output, add, norm
for the next sub-layer" as one kernel (csrc/norm.cu add_rms_norm), reaching
over to the next block's first norm when the model passes it.
"""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from ..config.spec import ConfigError
from .registry import register_block


def _fusable(norm) -> bool:
    return norm is None or getattr(norm, "fusable_rms", False)


class SandwichBlock:
    norm_sites = ("pre_mixer", "post_mixer", "pre_feed_forward", "post_feed_forward")
    required_sites = ("pre_mixer", "pre_feed_forward")

    def __init__(self, mixer, feed_forward, norms: Mapping[str, object], rt):
        for site in self.required_sites:
            if norms.get(site) is None:
                raise ConfigError(f"block: the '{site}' norm is required")
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.pre_mixer = norms["pre_mixer"]
        self.post_mixer = norms.get("post_mixer")
        self.pre_ff = norms["pre_feed_forward"]
        self.post_ff = norms.get("post_feed_forward")
        self.rt = rt

    @property
    def first_norm(self):
        return self.pre_mixer

    @property
    def chain_safe(self) -> bool:
        """Whether this block may run while few-row steps are deferred into a chain
        (parts/base.py Runtime.chaining): its mixer and feed-forward promise to touch
        deferred results through the runtime and ``kernels.native`` only, and its norms are
        the kind the residual kernel applies."""
        return (getattr(self.mixer, "chain_safe", False)
                and getattr(self.feed_forward, "chain_safe", False)
                and all(_fusable(n) for n in (self.pre_mixer, self.post_mixer, self.pre_ff,
                                              self.post_ff)))

    @property
    def captures_prompts(self) -> bool:
        """Whether a recorded step of prompts of this block may be replayed for other prompts:
        its mixer and feed-forward promise to read sequences, slots and counts on the
        device only (the block itself and the norms work row by row)."""
        return (getattr(self.mixer, "captures_prompts", False)
                and getattr(self.feed_forward, "captures_prompts", False))

    def _add_then_norm(self, y: torch.Tensor, post, h: torch.Tensor, nxt) -> Optional[torch.Tensor]:
        """h += post(y) (or y); returns nxt(h) if nxt is given."""
        if _fusable(post) and _fusable(nxt):
            out = torch.empty_like(y) if nxt is not None else None
            self.rt.add_rms_norm(y, post.gain if post is not None else None,
                                 post.eps if post is not None else 0.0, h,
                                 nxt.gain if nxt is not None else None,
                                 nxt.eps if nxt is not None else 0.0, out)
            return out
        self.rt.flush()         # the steps below read y and h outside the chain
        if post is not None:
            y = post.forward(y, out_dtype=torch.float32)
        h.add_(y.to(torch.float32))
        return nxt.forward(h, out_dtype=self.rt.dtype) if nxt is not None else None

    def forward(self, h: torch.Tensor, normed: Optional[torch.Tensor], ctx, entry: int,
                cache_entry: int, owns_cache: bool, next_norm=None) -> Optional[torch.Tensor]:
        if normed is None:
            self.rt.flush()
            normed = self.pre_mixer.forward(h, out_dtype=self.rt.dtype)
        a = self.mixer.forward(normed, ctx, entry, cache_entry, owns_cache)
        n2 = self._add_then_norm(a, self.post_mixer, h, self.pre_ff)
        f = self.feed_forward.forward(n2, ctx)
        return self._add_then_norm(f, self.post_ff, h, next_norm)


class PreNormBlock(SandwichBlock):
    norm_sites = ("pre_mixer", "pre_feed_forward")


register_block("sandwich", SandwichBlock)
register_block("pre_norm", PreNormBlock)
