"""Oracle: next-token sampling (test infrastructure).

Restates sample (examples/llm/qwen3.py:395-418) with one change that makes it checkable
outside JAX: the categorical draw is the inverse CDF at a caller-supplied uniform number
instead of jax.random.categorical's Gumbel noise.  Candidate order is the reference's: the
whole row in vocabulary order when neither top_k nor top_p is set, else the top_k values in
descending order (ties: lower index first), cut by top_p to the smallest prefix whose
probability reaches top_p.  Also returns how far u * total lies from the nearest CDF step
(as a fraction of the total), so that a test can skip draws that f32 rounding could move."""
import numpy as np


def sample(logits, u, temperature=0.0, top_k=0, top_p=1.0):
    logits = np.asarray(logits, np.float64)
    B, V = logits.shape
    if temperature < 0:
        raise ValueError("temperature must be >= 0")
    if not 0 <= top_k <= V:
        raise ValueError("top_k out of range")
    out = np.zeros(B, np.int32)
    margin = np.full(B, np.inf)
    for r in range(B):
        x = logits[r]
        if temperature == 0.0:
            out[r] = int(np.argmax(x))
            continue
        z = x / temperature
        if not top_k and top_p >= 1.0:
            idx = np.arange(V)
            vals = z
        else:
            order = np.lexsort((np.arange(V), -z))          # descending value, ties by lower index
            idx = order[:top_k] if top_k else order
            vals = z[idx]
            if top_p < 1.0:
                p = np.exp(vals - vals.max())
                p /= p.sum()
                before = np.cumsum(p) - p
                keep = before < top_p
                keep[0] = True
                idx, vals = idx[keep], vals[keep]
        p = np.exp(vals - z.max())
        cdf = np.cumsum(p)
        target = u[r] * cdf[-1]
        j = int(np.searchsorted(cdf, target, side="right"))
        j = min(j, len(idx) - 1)
        out[r] = idx[j]
        edges = np.concatenate([[0.0], cdf])
        margin[r] = np.min(np.abs(edges - target)) / cdf[-1]
    return out, margin
