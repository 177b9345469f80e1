"""From the logits of a step to one token per row, on the device."""
from __future__ import annotations

import numpy as np
import torch

from .params import SamplingParams

_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform_for(seed: int, index: int) -> float:
    """A number in [0, 1) that depends on (seed, index of the generated token) only: the
    same request draws the same tokens whatever else is in the batch and however its
    prompt was cut."""
    h = _splitmix64(_splitmix64(seed & _MASK) ^ ((index * 0xD6E8FEB86659FD93) & _MASK))
    return (h >> 40) * (1.0 / (1 << 24))


class Sampler:
    """Batches the rows of a step: processors in place on the logits, one filter launch
    when any row filters, one sampling launch for all rows."""

    def __init__(self, rt):
        self.rt = rt

    def sample(self, logits: torch.Tensor, rows: list[tuple[SamplingParams, int, int, list[int]]]) -> torch.Tensor:
        """rows[i] = (params, seed, index of the token being drawn, token history) for
        logits[i].  -> int32 [len(rows)] on the device."""
        k, dev = self.rt.k, self.rt.device
        n = len(rows)
        assert logits.shape[0] == n
        bias = [(i, t, v) for i, (p, _, _, _) in enumerate(rows) for t, v in p.logit_bias.items()]
        if bias:
            arr = np.array(bias, dtype=np.float64)
            k.logit_bias(logits, torch.from_numpy(arr[:, 0].astype(np.int32)).to(dev),
                         torch.from_numpy(arr[:, 1].astype(np.int32)).to(dev),
                         torch.from_numpy(arr[:, 2].astype(np.float32)).to(dev))
        H = max((p.history_needed for p, _, _, _ in rows), default=0)
        if H > 0:
            hist = np.full((n, H), -1, dtype=np.int32)
            pen = np.zeros((n, 3), dtype=np.float32)
            win = np.zeros((n, 3), dtype=np.int32)
            for i, (p, _, _, toks) in enumerate(rows):
                tail = toks[-H:]
                if tail:
                    hist[i, H - len(tail):] = tail
                pen[i] = (p.repetition_penalty if p.repetition_penalty != 0 else 1.0, p.presence_penalty,
                          p.frequency_penalty)
                win[i] = (p.repetition_context_size, p.presence_context_size, p.frequency_context_size)
            pen_d = torch.from_numpy(pen).to(dev)
            k.penalties(logits, torch.from_numpy(hist).to(dev), pen_d[:, 0].contiguous(), pen_d[:, 1].contiguous(),
                        pen_d[:, 2].contiguous(), torch.from_numpy(win).to(dev))
        if all(p.greedy for p, _, _, _ in rows):
            return k.sample(logits)
        par = np.zeros((4, n), dtype=np.float32)          # temperature, uniform, top_p, min_p
        ints = np.zeros((2, n), dtype=np.int32)           # top_k, min_tokens_to_keep
        for i, (p, seed, index, _) in enumerate(rows):
            par[0, i], par[1, i] = p.temperature, uniform_for(seed, index)
            if not p.greedy:                              # a greedy row has no filter
                par[2, i] = p.top_p if 0 < p.top_p < 1.0 else 0.0
                par[3, i] = p.min_p
                ints[0, i] = p.top_k
            ints[1, i] = p.min_tokens_to_keep
        par_d = torch.from_numpy(par).to(dev)
        keep = None
        if any(p.filters_on for p, _, _, _ in rows):
            ints_d = torch.from_numpy(ints).to(dev)
            keep = k.filter_mask(logits, par_d[2], par_d[3], ints_d[0], ints_d[1])
        return k.sample(logits, par_d[0], par_d[1], keep)
