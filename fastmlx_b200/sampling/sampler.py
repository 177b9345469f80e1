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


class _Upload:
    """One packed host-to-device copy per step for everything the sampling kernels read: a
    small ring of pinned buffers (a buffer is written again only after the copy that last
    read it has finished), so that the host never waits for the device here.  A pageable
    `.to(device)` would: it returns only when the stream has reached the copy, which puts
    the host in step with the device and undoes the engine's step ahead."""

    def __init__(self, device, ring: int = 4):
        self.device = device
        self.cuda = torch.device(device).type == "cuda"
        self.ring, self.at = ring, 0
        self.hosts: list = [None] * ring
        self.events: list = [None] * ring

    def send(self, arrays: list[np.ndarray]) -> list[torch.Tensor]:
        """int32 / float32 arrays -> device tensors of the same shapes and types (views of one
        device buffer; every array starts on a 16-byte boundary)."""
        offs, total = [], 0
        for a in arrays:
            total = (total + 3) // 4 * 4
            offs.append(total)
            total += a.size
        self.at = (self.at + 1) % self.ring
        host = self.hosts[self.at]
        if host is None or host.numel() < total:
            host = torch.empty(max(total, 1024), dtype=torch.int32)
            self.hosts[self.at] = host = host.pin_memory() if self.cuda else host
            self.events[self.at] = None
        if self.events[self.at] is not None:
            self.events[self.at].synchronize()
        flat = host.numpy()
        for a, o in zip(arrays, offs):
            flat[o: o + a.size] = a.reshape(-1).view(np.int32)
        dev = host[:total].to(self.device, non_blocking=True) if self.cuda else host[:total].clone()
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record()
            self.events[self.at] = ev
        out = []
        for a, o in zip(arrays, offs):
            t = dev[o: o + a.size]
            out.append((t.view(torch.float32) if a.dtype == np.float32 else t).view(a.shape))
        return out


class Sampler:
    """Batches the rows of a step: processors in place on the logits, one filter launch
    when any row filters, one sampling launch for all rows; one upload for their arguments."""

    def __init__(self, rt):
        self.rt = rt
        self.upload = _Upload(rt.device)

    def sample(self, logits: torch.Tensor, rows: list[tuple[SamplingParams, int, int, list[int]]]) -> torch.Tensor:
        """rows[i] = (params, seed, index of the token being drawn, token history) for
        logits[i].  -> int32 [len(rows)] on the device."""
        k = self.rt.k
        n = len(rows)
        assert logits.shape[0] == n
        arrays: list[np.ndarray] = []
        bias = [(i, t, v) for i, (p, _, _, _) in enumerate(rows) for t, v in p.logit_bias.items()]
        if bias:
            arr = np.array(bias, dtype=np.float64)
            arrays += [arr[:, 0].astype(np.int32), arr[:, 1].astype(np.int32), arr[:, 2].astype(np.float32)]
        H = max((p.history_needed for p, _, _, _ in rows), default=0)
        if H > 0:
            hist = np.full((n, H), -1, dtype=np.int32)
            pen = np.zeros((3, n), dtype=np.float32)
            win = np.zeros((n, 3), dtype=np.int32)
            for i, (p, _, _, toks) in enumerate(rows):
                tail = toks[-H:]
                if tail:
                    hist[i, H - len(tail):] = tail
                pen[:, i] = (p.repetition_penalty if p.repetition_penalty != 0 else 1.0, p.presence_penalty,
                             p.frequency_penalty)
                win[i] = (p.repetition_context_size, p.presence_context_size, p.frequency_context_size)
            arrays += [hist, pen, win]
        greedy = all(p.greedy for p, _, _, _ in rows)
        filters = not greedy and any(p.filters_on for p, _, _, _ in rows)
        if not greedy:
            par = np.zeros((4, n), dtype=np.float32)          # temperature, uniform, top_p, min_p
            ints = np.zeros((2, n), dtype=np.int32)           # top_k, min_tokens_to_keep
            for i, (p, seed, index, _) in enumerate(rows):
                par[0, i], par[1, i] = p.temperature, uniform_for(seed, index)
                if not p.greedy:                              # a greedy row has no filter
                    par[2, i] = p.top_p if 0 < p.top_p < 1.0 else 0.0
                    par[3, i] = p.min_p
                    ints[0, i] = p.top_k
                ints[1, i] = p.min_tokens_to_keep
            arrays += [par, ints]
        dev = self.upload.send(arrays) if arrays else []
        if bias:
            k.logit_bias(logits, dev[0], dev[1], dev[2])
            dev = dev[3:]
        if H > 0:
            hist_d, pen_d, win_d = dev[:3]
            k.penalties(logits, hist_d, pen_d[0], pen_d[1], pen_d[2], win_d)
            dev = dev[3:]
        if greedy:
            return k.sample(logits)
        par_d, ints_d = dev
        if hasattr(k, "filter_sample") and k.filter_sample_takes(logits.shape[1]):
            # wide rows: filters and draw in one kernel, a row on a cluster of 8 blocks, no mask in memory
            if filters:
                return k.filter_sample(logits, par_d[0], par_d[1], par_d[2], par_d[3], ints_d[0], ints_d[1])
            if 8 * n <= k.num_sms(logits.device):
                # without filters only while the rows' clusters run at once (8 rows of 128,256 logits: 17 us against
                # 35 on one block per row; 64 rows: 80 against 40)
                return k.filter_sample(logits, par_d[0], par_d[1])
        keep = k.filter_mask(logits, par_d[2], par_d[3], ints_d[0], ints_d[1]) if filters else None
        return k.sample(logits, par_d[0], par_d[1], keep)
