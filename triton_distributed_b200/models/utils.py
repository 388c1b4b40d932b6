"""Sampling, seeding and logging helpers (reference: ``python/triton_dist/models/utils.py:42-96``)."""
from __future__ import annotations

import logging
import random
import sys

import numpy as np
import torch


def seed_everything(seed: int = 0) -> None:
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def sample_token(logits: torch.Tensor, temperature: float = 0.6, top_p: float = 0.95) -> torch.Tensor:
    """Top-p (nucleus) sampling; ``temperature == 0`` is greedy. logits [B, 1|S, V] -> token ids [B, 1]."""
    logits = logits[:, -1, :].float() if logits.dim() == 3 else logits.float()
    if temperature <= 0.0:
        return logits.argmax(-1, keepdim=True)
    if logits.is_cuda:
        from .. import ops
        return ops.top_p_sample(logits, temperature, top_p)
    probs = torch.softmax(logits / temperature, dim=-1)
    sp, si = torch.sort(probs, dim=-1, descending=True)
    keep = (torch.cumsum(sp, -1) - sp) < top_p
    sp = sp * keep
    sp = sp / sp.sum(-1, keepdim=True)
    choice = torch.multinomial(sp, 1)
    return si.gather(-1, choice)


class _Formatter(logging.Formatter):
    COLORS = {logging.DEBUG: "\033[36m", logging.INFO: "\033[32m", logging.WARNING: "\033[33m", logging.ERROR: "\033[31m"}

    def format(self, record):
        c = self.COLORS.get(record.levelno, "") if sys.stderr.isatty() else ""
        end = "\033[0m" if c else ""
        return f"{c}[{self.formatTime(record, '%H:%M:%S')}] {record.levelname}{end} {record.getMessage()}"


def _make_logger() -> logging.Logger:
    lg = logging.getLogger("b200dist")
    if not lg.handlers:
        h = logging.StreamHandler()
        h.setFormatter(_Formatter())
        lg.addHandler(h)
        lg.setLevel(logging.INFO)
        lg.propagate = False
    return lg


logger = _make_logger()
