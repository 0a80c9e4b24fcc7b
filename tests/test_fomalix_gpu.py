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
