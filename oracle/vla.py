"""CPU oracle of the GR00T-N1.5-shaped vision-language-action model (TEST INFRASTRUCTURE; see oracle/__init__.py):
the Qwen2.5-VL-shaped FP8 prefill of ``oracle/qwen_vl.py`` followed by the flow-matching action head of
``oracle/dit.py`` cross-attending to the prefill's final hidden states, as ``aginfer_b200/recipes/vla.py`` lays
them out.  The reference project has no implementation of either (parity unpinned)."""
from __future__ import annotations

import torch

from . import dit, qwen_vl


def forward(cfg, w: dict, pixels, input_ids, positions, state, noise) -> tuple[torch.Tensor, torch.Tensor]:
    """Returns (actions [horizon, action_dim] fp32, hidden_out [tokens, hidden] bf16)."""
    hidden, _ = qwen_vl.forward(cfg.backbone, w, pixels, input_ids, positions)
    return dit.forward(cfg.head, w, hidden, state, noise), hidden
