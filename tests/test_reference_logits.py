"""The plain implementation against logits that the REFERENCE engine itself computed.

``tests/golden/reference_logits_<model>.npy`` were written on a B200 by the reference's own
``Engine::score`` (its CUDA kernels and cuBLAS, fp16 storage), built unmodified for sm_100a, on the
small random models of ``tests/golden/golden_models.py`` (``tests/golden/make_reference_logits.py``
says how).  The plain implementation of this test suite -- the oracle of every replay test -- must
agree with them: run with the reference's roundings (``storage=float16``) it may differ only by what
those roundings leave open (fp16 products of cuBLAS against float64 sums rounded once).

The bound is the reference's own: against float32 logits of the original model its documentation
reports a mean absolute error of 0.0023 and a maximum of 0.0148 (``docs/design.md:131``).
"""
import os
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import golden_models as gm  # noqa: E402
import plain_llama  # noqa: E402

REFERENCE_MAX_ERROR = 0.0148
REFERENCE_MEAN_ERROR = 0.0023


@pytest.mark.parametrize("name", sorted(gm.MODELS))
def test_plain_implementation_matches_the_reference_engine(name):
    m = gm.MODELS[name]
    golden = torch.from_numpy(np.load(os.path.join(HERE, "golden", f"reference_logits_{name}.npy"))).double()
    w = {k: torch.from_numpy(v.astype(np.float64)) for k, v in gm.tensors(name).items()}
    toks = gm.token_ids(m["seed"], m["tokens"], m["cfg"]["vocab_size"])
    ours = plain_llama.llama_forward(m["cfg"], w, toks, storage=torch.float16)[-m["keep"]:]
    assert ours.shape == golden.shape
    d = (ours - golden).abs()
    assert d.max().item() <= REFERENCE_MAX_ERROR, f"{name}: max |d| {d.max().item():.4f}"
    assert d.mean().item() <= REFERENCE_MEAN_ERROR, f"{name}: mean |d| {d.mean().item():.5f}"
    # And the logits are not near zero, where any two implementations would agree.
    assert golden.std().item() > 0.2
    # The greedy pick agrees wherever the reference's own margin exceeds the bound.
    top2 = golden.topk(2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 2 * REFERENCE_MAX_ERROR
    assert clear.sum() > m["keep"] // 2
    assert (ours.argmax(-1)[clear] == golden.argmax(-1)[clear]).all()


def test_a_wrong_formula_would_show():
    """The bound separates the plain implementation from near misses: the interleaved rotary
    pairing, a missing 1/sqrt(hd), the weight multiplied before the rounding."""
    name = "hd128_g4"
    m = gm.MODELS[name]
    golden = torch.from_numpy(np.load(os.path.join(HERE, "golden", f"reference_logits_{name}.npy"))).double()
    w = {k: torch.from_numpy(v.astype(np.float64)) for k, v in gm.tensors(name).items()}
    toks = gm.token_ids(m["seed"], m["tokens"], m["cfg"]["vocab_size"])
    cfg = dict(m["cfg"], rope_theta=m["cfg"]["rope_theta"] * 1.5)
    off = plain_llama.llama_forward(cfg, w, toks, storage=torch.float16)[-m["keep"]:]
    assert (off - golden).abs().max().item() > REFERENCE_MAX_ERROR
    cfg = dict(m["cfg"], rms_norm_eps=1e-2)
    off = plain_llama.llama_forward(cfg, w, toks, storage=torch.float16)[-m["keep"]:]
    assert (off - golden).abs().max().item() > REFERENCE_MAX_ERROR
