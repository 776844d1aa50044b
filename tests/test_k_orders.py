"""Activation K orders of the two packed-weight GEMMs: the index maps that producers and tests use (CPU)."""
import torch

from oxibonsai_b200.ops import cuda_ops as K


def test_paired_k_index_is_a_permutation_inside_every_16_inputs():
    k = 256
    perm = K.paired_k_index(k)
    assert sorted(perm.tolist()) == list(range(k))
    assert torch.equal(perm // 16, torch.arange(k) // 16)                 # nothing leaves its 16-input word
    assert torch.equal((perm & 8), (torch.arange(k) & 8))                 # nor its half of the word (the a / b planes)
    # inside a half: inputs p and p + 4 sit side by side (one half2 of the expanded weights)
    j = torch.arange(8)
    assert perm[:8].tolist() == ((j & 3) * 2 + ((j >> 2) & 1)).tolist()
    assert perm[0] + 1 == perm[4] and perm[3] + 1 == perm[7]


def test_hmma_k_index_is_a_permutation_inside_every_128_inputs():
    k = 384
    perm = K.hmma_k_index(k)
    assert sorted(perm.tolist()) == list(range(k))
    assert torch.equal(perm // 128, torch.arange(k) // 128)
    # one MMA k-step (16 consecutive positions) holds, for the four words 2c + j of a lane column c, the weights
    # {p, p + 4} of plane a then of plane b: positions 0..15 of step (j = 0, p = 0) come from inputs with e in {0, 4, 8, 12}
    step0 = [int(i) for i in range(128) if perm[i] < 16]
    assert all((i & 15) in (0, 4, 8, 12) for i in step0) and len(step0) == 16
    # a natural-order row scattered with the map and gathered back is unchanged
    x = torch.randn(3, k)
    y = torch.empty_like(x)
    y[:, perm] = x
    assert torch.equal(y[:, perm], x)
