"""Two sequence mixers side by side on the same input.  ``combine = "normed_mean"``: each output is RMS-normed over the
model width with its own plain weight and the layer's result is half their sum; the norms and the mean are left to the
layer's output norm (``norms.OutputRMSNormAdd`` takes the ``BranchPair`` returned here and does all of it in one kernel).
``combine = "scaled_sum"``: the result is ``left_scale * left + right_scale * right``, left to the layer's stream connection
(``norms.StreamConnection`` takes the ``ScaledPair`` returned here)."""
from __future__ import annotations

import torch
import torch.nn as nn

from .module import MegatronModule
from .norms import BranchPair, ScaledPair


class SideBySideMixer(MegatronModule):
    def __init__(self, config, layer_number: int, left: nn.Module, right: nn.Module, combine: str = "normed_mean",
                 left_scale: float = 1.0, right_scale: float = 1.0):
        super().__init__(config)
        if combine not in ("normed_mean", "scaled_sum"):
            raise ValueError(f"unknown combination {combine!r}")
        self.layer_number = layer_number
        self.left, self.right = left, right
        self.combine, self.left_scale, self.right_scale = combine, float(left_scale), float(right_scale)
        if combine == "normed_mean":
            dev = "cpu" if (config.use_cpu_initialization or not torch.cuda.is_available()) else torch.cuda.current_device()
            self.left_out_weight = nn.Parameter(torch.ones(config.hidden_size, dtype=config.params_dtype, device=dev))
            self.right_out_weight = nn.Parameter(torch.ones(config.hidden_size, dtype=config.params_dtype, device=dev))

    def forward(self, hidden_states, inference_context=None, cache_index=None, **kw):
        a, bias_a = self.left(hidden_states, inference_context=inference_context, cache_index=cache_index, **kw)
        b, bias_b = self.right(hidden_states, inference_context=inference_context, cache_index=cache_index, **kw)
        if self.combine == "scaled_sum":
            if bias_b is not None:
                b = b + bias_b
            return ScaledPair(a, b, bias_a, self.left_scale, self.right_scale), None
        if bias_a is not None:
            a = a + bias_a
        if bias_b is not None:
            b = b + bias_b
        return BranchPair(a, b, self.left_out_weight, self.right_out_weight), None
