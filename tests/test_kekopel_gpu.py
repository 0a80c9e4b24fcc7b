"""The Kekopel cases of ``test_kekopel.py`` on the CUDA kernels (``csrc/seq_mixers.cu``, ``csrc/moe_ragged.cu``): the same
functions, collected here under the ``gpu`` marker; the ops take their kernel branch because their tensors live on the
device."""
import pytest
import torch

from test_kekopel import *  # noqa: F401,F403  (collects every test of that module again)
from test_kekopel import MIXED, O, feed, make_engine, tokens
from shuffle_exchange_b200.native import lib as _lib

pytestmark = pytest.mark.gpu


def test_the_kernels_ran():
    before = _lib.launch_count
    from shuffle_exchange_b200.inference.v2.kernels import mixer_ops as M
    x = torch.randn(3, 10, device="cuda")
    out = M.rms_scale_rows(x, None, torch.tensor([2.0], device="cuda"), 1e-6, torch.float32)
    assert _lib.launch_count == before + 1
    assert torch.allclose(out.pow(2).mean(-1), torch.full((3,), 4.0, device="cuda"), atol=1e-3)


def test_experts_on_the_grouped_gemm_path():
    """Widths that are multiples of 64 in bf16 take the grouped tensor-core path with the routing weight applied while
    the rows are moved; prompts of more than 16 tokens take the tiled attention kernel."""
    layers = [dict(MIXED["layers"][0], mlp={"expert": {"ff": 32}, "kind": "moe", "router": {"experts": 4, "top": 2}}),
              dict(MIXED["layers"][1], mlp={"expert": {"ff": 64}, "kind": "moe", "router": {"experts": 3, "top": 1}})]
    cfg = dict(MIXED, layers=layers, width=64)
    W = O.random_weights(cfg, seed=31)
    toks = tokens(70, cfg["vocab"], 32)
    want = O.forward(toks, W, cfg)[0]
    eng = make_engine(cfg, W, dtype=torch.bfloat16)
    for sizes in ([len(toks)], [33, 1, 17, 1, 1]):
        d = feed(eng, len(sizes), toks, sizes) - want
        err = (d - d.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt() / want.std()
        # a token whose two best experts score nearly alike may be routed otherwise in 16-bit: a few rows may differ
        assert err.median() < 0.02 and (err > 0.08).sum() <= 7, err


def test_other_sizes_in_bf16():
    """Widths, ranks and head sizes that are not multiples of 8 take the scalar forms of the kernels and the library
    products; 16-bit serving must still follow the exact evaluation."""
    from test_kekopel import ODD
    for cfg in ODD:
        W = O.random_weights(cfg, seed=8)
        toks = tokens(40, cfg["vocab"], 9)
        want = O.forward(toks, W, cfg)[0]
        eng = make_engine(cfg, W, dtype=torch.bfloat16, block_size=8)
        for uid, sizes in ((1, [len(toks)]), (2, [19, 1, 2])):
            d = feed(eng, uid, toks, sizes) - want
            err = (d - d.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt() / want.std()
            assert err.median() < 0.03 and (err > 0.12).sum() <= 4, err
