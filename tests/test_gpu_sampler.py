"""GPU sampler: tie rule, top-k / top-p semantics, distribution of draws, on-device RNG state."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _xorshift(x):
    m = (1 << 64) - 1
    x ^= (x << 13) & m
    x ^= x >> 7
    x ^= (x << 17) & m
    return x


def _reference_sample(logits, T, k, p, state):
    """The reference algorithm on the host (sort order made deterministic: descending prob, ascending index)."""
    v = logits.astype(np.float32) / np.float32(T)
    idx = np.arange(len(v))
    if 0 < k < len(v):
        order = np.lexsort((idx, -v))[:k]
        idx, v = idx[order], v[order]
    e = np.exp(v - v.max()).astype(np.float32)
    pr = e / e.sum()
    order = np.lexsort((idx, -pr))
    idx, pr = idx[order], pr[order]
    if p < 1.0:
        cum = np.cumsum(pr)
        cut = int(np.argmax(cum > p)) if (cum > p).any() else len(pr) - 1
        idx, pr = idx[: cut + 1], pr[: cut + 1]
        pr = pr / pr.sum()
    state = _xorshift(state)
    r = np.float32(state / float((1 << 64) - 1))
    cum = np.cumsum(pr)
    hit = np.nonzero(r <= cum)[0]
    return int(idx[hit[0]] if len(hit) else idx[0]), state, set(idx.tolist())


def test_greedy_returns_last_maximum_and_advances():
    from oxibonsai_b200.ops import cuda_ops as K
    lg = torch.zeros((3, 151936), device=DEV)
    lg[0, 17] = 5; lg[0, 90000] = 5; lg[0, 151935] = 5
    lg[1, 1234] = 2.0
    lg[2] = -1.0  # all tied: last index wins
    pos = torch.tensor([4, 5, 6], dtype=torch.int32, device=DEV)
    out = K.sample(lg, positions=pos, advance=True)
    assert out.tolist() == [151935, 1234, 151935] and pos.tolist() == [5, 6, 7]
    temps = torch.zeros(3, device=DEV)
    rng = torch.ones(3, dtype=torch.int64, device=DEV)
    assert K.sample(lg, temps, torch.zeros(3, dtype=torch.int32, device=DEV), torch.ones(3, device=DEV), rng).tolist() == [151935, 1234, 151935]


@pytest.mark.parametrize("T,k,p", [(0.7, 40, 0.9), (0.2, 10, 0.8), (1.0, 5, 1.0), (0.8, 50, 0.9), (0.1, 10, 0.5)])
def test_topk_path_matches_reference_token_by_token(T, k, p):
    from oxibonsai_b200.ops import cuda_ops as K
    g = torch.Generator().manual_seed(11)
    vocab = 151936
    lg = torch.randn((1, vocab), generator=g) * 3
    lgd = lg.to(DEV)
    temps, topks, topps = (torch.tensor([x], dtype=d, device=DEV) for x, d in ((T, torch.float32), (k, torch.int32), (p, torch.float32)))
    rng = torch.tensor([42], dtype=torch.int64, device=DEV)
    state = 42
    for _ in range(40):
        tok = K.sample(lgd, temps, topks, topps, rng).item()
        ref, state, allowed = _reference_sample(lg[0].numpy(), T, k, p, state)
        assert tok in allowed
        assert tok == ref
        assert (rng.item() & ((1 << 64) - 1)) == state


def test_full_vocab_path_respects_top_p_and_distribution():
    from oxibonsai_b200.ops import cuda_ops as K
    vocab = 5000
    g = torch.Generator().manual_seed(12)
    lg = torch.randn((1, vocab), generator=g) * 4
    T, p = 1.0, 0.95
    pr = torch.softmax(lg[0].double() / T, -1)
    srt, order = torch.sort(pr, descending=True)
    cum = torch.cumsum(srt, 0)
    cut = int((cum > p).nonzero()[0])
    allowed = set(order[: cut + 1].tolist())
    lgd = lg.to(DEV)
    temps, topks, topps = torch.tensor([T], device=DEV), torch.tensor([0], dtype=torch.int32, device=DEV), torch.tensor([p], device=DEV)
    rng = torch.tensor([7], dtype=torch.int64, device=DEV)
    draws = [K.sample(lgd, temps, topks, topps, rng).item() for _ in range(3000)]
    assert set(draws) <= allowed
    # the most likely token should be drawn about pr[top] / kept_mass of the time
    top = int(order[0])
    expect = float(srt[0] / cum[cut])
    freq = draws.count(top) / len(draws)
    assert abs(freq - expect) < 4 * np.sqrt(expect * (1 - expect) / len(draws)) + 0.01
    # top_p = 1: every token possible, mean log-prob of draws close to the negative entropy
    topps.fill_(1.0)
    draws = torch.tensor([K.sample(lgd, temps, topks, topps, rng).item() for _ in range(3000)])
    ent = -(pr * pr.log()).sum().item()
    assert abs(-pr.log()[draws].mean().item() - ent) < 0.25


def test_allow_mask_constrains_every_path():
    from oxibonsai_b200.ops import cuda_ops as K
    vocab = 1000
    lg = torch.randn((1, vocab), generator=torch.Generator().manual_seed(13)).to(DEV)
    allowed = [3, 500, 999]
    mask = torch.zeros((1, (vocab + 31) // 32), dtype=torch.int32, device=DEV)
    for a in allowed:
        mask[0, a // 32] |= (1 << (a % 32)) if a % 32 != 31 else -(1 << 31)
    rng = torch.tensor([5], dtype=torch.int64, device=DEV)
    best = max(allowed, key=lambda a: lg[0, a].item())
    assert K.sample(lg, allow_mask=mask).item() == best
    for k in (0, 2, 40):
        temps, topks, topps = torch.tensor([1.5], device=DEV), torch.tensor([k], dtype=torch.int32, device=DEV), torch.tensor([1.0], device=DEV)
        for _ in range(50):
            assert K.sample(lg, temps, topks, topps, rng, allow_mask=mask).item() in allowed
