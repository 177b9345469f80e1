"""Plain statements of the sampling filters and logits processors, from the formulas of
tamnd/fastmlx compute/sampler.go and compute/logits_processor.go (each function cites its
lines).  Rows are Python lists; nothing here is shared with the package."""
import math

NEG_INF = float("-inf")


def log_softmax(row):
    m = max(row)
    lse = m + math.log(sum(math.exp(v - m) for v in row))
    return [v - lse for v in row]


def top_p_keep(logprobs, top_p):
    """compute/sampler.go:79-108: ascending stable order, running mass, keep where the mass
    up to and including the token exceeds 1 - top_p."""
    order = sorted(range(len(logprobs)), key=lambda i: logprobs[i])       # stable
    run, cum = 0.0, [0.0] * len(logprobs)
    for i in order:
        run += math.exp(logprobs[i])
        cum[i] = run
    return [c > 1.0 - top_p for c in cum]


def top_indices(row, k):
    """compute/sampler.go:155-173: the k largest, equal values by lower index."""
    return sorted(range(len(row)), key=lambda i: (-row[i], i))[:k]


def min_p_keep(row, min_p, min_keep=1):
    """compute/sampler.go:114-135."""
    if not (0 < min_p <= 1.0):
        return [True] * len(row)
    floor = max(row) + math.log(min_p)
    keep = [not (v < floor) for v in row]
    if min_keep > 1:
        for i in top_indices(row, min_keep):
            keep[i] = True
    return keep


def top_k_keep(row, k):
    """compute/sampler.go:139-153."""
    if k <= 0 or k >= len(row):
        return [True] * len(row)
    idx = set(top_indices(row, k))
    return [i in idx for i in range(len(row))]


def apply_filters(logits, top_p=0.0, min_p=0.0, top_k=0, min_keep=1):
    """compute/sampler.go:46-59: top-p, then min-p, then top-k, each on what the one before
    left (masked tokens are -inf).  -> keep list."""
    row = log_softmax(logits)
    keep = [True] * len(row)

    def mask(k2):
        for i, kk in enumerate(k2):
            if not kk:
                keep[i] = False
                row[i] = NEG_INF

    if 0 < top_p < 1.0:
        mask(top_p_keep(row, top_p))
    if min_p != 0.0:
        mask(min_p_keep(row, min_p, min_keep))
    if 0 < top_k < len(row):
        mask(top_k_keep(row, top_k))
    return keep


def window(tokens, n):
    return tokens[-n:] if n > 0 and len(tokens) > n else tokens


def apply_processors(tokens, logits, logit_bias=None, repetition=None, presence=None, frequency=None,
                     rep_ctx=20, pres_ctx=20, freq_ctx=20):
    """compute/logits_processor.go:61-164, in its order.  32-bit arithmetic is imitated with
    struct round trips where the fixture pins it."""
    import struct
    f32 = lambda x: struct.unpack("f", struct.pack("f", x))[0]
    row = [f32(v) for v in logits]
    if logit_bias:
        for i, v in logit_bias.items():
            if 0 <= int(i) < len(row):
                row[int(i)] = f32(row[int(i)] + f32(v))
    if repetition is not None and repetition != 0 and tokens:
        p = f32(repetition)
        for t in dict.fromkeys(window(tokens, rep_ctx)):
            if 0 <= t < len(row):
                row[t] = f32(row[t] * p) if row[t] < 0 else f32(row[t] / p)
    if presence is not None and presence != 0 and tokens:
        for t in dict.fromkeys(window(tokens, pres_ctx)):
            if 0 <= t < len(row):
                row[t] = f32(row[t] - f32(presence))
    if frequency is not None and frequency != 0 and tokens:
        for t in window(tokens, freq_ctx):
            if 0 <= t < len(row):
                row[t] = f32(row[t] - f32(frequency))
    return row
