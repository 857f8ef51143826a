"""Regenerates the golden fixtures in this folder from the CPU checker (oracle/gdn_oracle.py, fp64).

The reference project holds no vectors for this path, so these fixtures pin the checker against drift,
not against the reference: parity stays "unpinned by the reference".  Run from the repository root:

    python tests/golden/make_golden.py
"""
import hashlib
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from avelang_b200 import synth  # noqa: E402
from oracle import gdn_oracle as O  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def small_case():
    """bf16 GQA case with a ragged varlen split, nonzero initial states, z and a slow gate."""
    inp = synth.make_inputs(1, 200, 2, 4, 64, 64, seed=7, with_z=True, n_states=3, gate_scale=0.05)
    inp.cu_seqlens = torch.tensor([0, 70, 71, 200], dtype=torch.int32)
    return inp


def main():
    c0 = synth.config0()
    o, s = O.naive_recurrent_gated_delta_rule(c0.q, c0.k, c0.v, c0.g, c0.beta, c0.scale)
    np.savez_compressed(os.path.join(HERE, "config0_fp64.npz"), o=o.float().numpy(), final_state=s.float().numpy(),
                        input_sha=np.array([sha(c0.q), sha(c0.k), sha(c0.v), sha(c0.g), sha(c0.beta)]))
    sm = small_case()
    o, s = O.naive_recurrent_gated_delta_rule(sm.q, sm.k, sm.v, sm.g, sm.beta, sm.scale, sm.initial_state, sm.cu_seqlens)
    y = O.gated_rmsnorm(o, sm.z)
    np.savez_compressed(os.path.join(HERE, "small_varlen_fp64.npz"), o=o.float().numpy(), y=y.float().numpy(),
                        final_state=s.float().numpy(),
                        input_sha=np.array([sha(sm.q), sha(sm.k), sha(sm.v), sha(sm.g), sha(sm.beta), sha(sm.z),
                                            sha(sm.initial_state)]))
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    main()
