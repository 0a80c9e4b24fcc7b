"""The Fomalix cases of ``test_fomalix.py`` on the CUDA kernels (``csrc/seq_mixers.cu``): the same functions, collected
here under the ``gpu`` marker; the ops take their kernel branch because their tensors live on the device."""
import pytest
import torch

from test_fomalix import *  # noqa: F401,F403  (collects every test of that module again)
from shuffle_exchange_b200.native import lib as _lib

pytestmark = pytest.mark.gpu


def test_the_kernels_ran():
    before = _lib.launch_count
    x = torch.randn(3, 10, device="cuda")
    from shuffle_exchange_b200.inference.v2.kernels import mixer_ops as M
    M.unit_norm_heads(x, 0, 2, 5, 1.0, 1e-6)
    assert _lib.launch_count == before + 1
    assert torch.allclose(x.view(3, 2, 5).pow(2).sum(-1), torch.ones(3, 2, device="cuda"), atol=1e-4)


@pytest.mark.parametrize("d,dv,chunk,sink", [(8, 12, 0, True), (64, 100, 37, True), (128, 128, 64, False), (20, 72, 5, True)])
def test_tiled_attention_equals_one_warp_per_query(d, dv, chunk, sink):
    """Atoms of 128, 100 and 3 queries of two sequences (the second continues at position 50): tiled and per-query
    kernels against the per-query kernel alone, fp32 and bf16 caches."""
    from shuffle_exchange_b200.inference.v2.kernels import mixer_ops as M
    g = torch.Generator().manual_seed(d)
    Hq, G, bs = 4, 2, 16
    lens, seen = [228, 3], [0, 50]
    T = sum(lens)
    q = torch.randn(T, Hq, d, generator=g).cuda()
    n_pages = 32
    for dt in (torch.float32, torch.bfloat16):
        kc = torch.randn(n_pages, bs, G, d, generator=g).to(dt).cuda()
        vc = torch.randn(n_pages, bs, G, dv, generator=g).to(dt).cuda()
        tables = torch.randperm(n_pages, generator=g).to(torch.int32).view(2, 16).cuda()
        t2s = torch.tensor([0] * lens[0] + [1] * lens[1], dtype=torch.int32).cuda()
        pos = torch.tensor(list(range(228)) + [50, 51, 52], dtype=torch.int32).cuda()
        atoms = torch.tensor([[0, 0, 128, 0, 0, 128], [0, 128, 100, 128, 0, 228], [1, 228, 3, 50, 0, 53]],
                             dtype=torch.int32).cuda()
        sk = torch.tensor([0.3, -1.0, 2.0, 0.0]).cuda() if sink else None
        ref = M.sink_attention(q, kc, vc, sk, t2s, pos, tables, d ** -0.5, chunk, dt).float()
        got = M.sink_attention(q, kc, vc, sk, t2s, pos, tables, d ** -0.5, chunk, dt, atoms, 2).float()
        tol = 2e-5 if dt == torch.float32 else 2e-2
        assert torch.allclose(got, ref, atol=tol, rtol=1e-4), float((got - ref).abs().max())
