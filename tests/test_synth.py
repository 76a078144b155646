"""The torch quantizers the benchmark builds its synthetic planes with must
produce the same bytes as the CPU oracle's restatement of the recipes."""
import numpy as np
import torch

import oracle
from paddock_b200 import synth


def test_q8_0_bytes_match_oracle():
    w = oracle.fill_normal(32 * 512, 3, 0.02)
    got = synth.quantize_q8_0(torch.from_numpy(w)).numpy()
    assert np.array_equal(got, oracle.quantize_q8_0(w))


def test_q4_k_bytes_match_oracle():
    w = oracle.fill_normal(256 * 300, 4, 0.02)
    w[:256] = 0.0            # an all-zero super-block
    w[256:512] = np.abs(w[256:512])  # an all-positive one (min clamps to 0)
    got = synth.quantize_q4_k(torch.from_numpy(w)).numpy()
    assert np.array_equal(got, oracle.quantize_q4_k(w))
