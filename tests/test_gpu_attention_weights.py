"""The attention matrix returned for debugging (return_attention=True of the forward launchers) against the oracle's."""
import numpy as np
import pytest
import torch

from oracle import sb_oracle as orc
from util import TOL_F32, rounded, synth, to_dev

pytestmark = pytest.mark.gpu


def _oracle_blocks(q, k, lengths, inv_temp, attend_current):
    """[H, T, T] block-diagonal float64 attention matrix of a pack."""
    H, T, _ = q.shape
    w = np.zeros((H, T, T))
    s = 0
    for n in lengths:
        _, _, att, _ = orc.sb_dense_fwd(q[:, s:s + n], k[:, s:s + n], k[:, s:s + n], inv_temp, attend_current,
                                        np.float64, return_att=True)
        w[:, s:s + n, s:s + n] = att
        s += n
    return w


@pytest.mark.parametrize("dtype,D,attend_current,cu_dtype", [
    (torch.float32, 40, False, torch.int64),
    (torch.bfloat16, 128, True, torch.int32),
    (torch.float16, 64, False, torch.int64),
])
def test_varlen_weights(dtype, D, attend_current, cu_dtype):
    from stickbreaking_attention_b200 import ops
    lengths = [70, 1, 33, 0, 130]
    H, T = 3, sum(lengths)
    q, k, v, _, _ = synth(H, T, D, 5)
    q, k, v = (rounded(x, dtype) for x in (q, k, v))
    inv_temp = 1.0 / np.sqrt(D)
    cu = torch.tensor(np.cumsum(lengths), dtype=cu_dtype, device="cuda")
    res = ops.varlen_fwd(to_dev(q, dtype), to_dev(k, dtype), to_dev(v, dtype), cu, max(lengths), inv_temp,
                         attend_current=attend_current, no_grad=True, return_attention=True)
    assert len(res) == 5
    o, rem, w = res[0], res[1], res[4]
    assert w.shape == (H, T, T) and w.dtype == torch.float32
    want = _oracle_blocks(q, k, lengths, inv_temp, attend_current)
    assert np.abs(w.double().cpu().numpy() - want).max() <= TOL_F32
    # the matrix explains the other two results: o = w v, rem = 1 - row sums
    tol = TOL_F32 if dtype == torch.float32 else 2e-2
    assert (torch.matmul(w, to_dev(v, torch.float32)) - o.float()).abs().max().item() <= tol
    assert ((1 - w.sum(-1)) - rem.float()).abs().max().item() <= tol


def test_batched_weights():
    from stickbreaking_attention_b200 import ops
    B, H, T, D = 2, 2, 97, 64
    g = torch.Generator().manual_seed(9)
    q, k, v = (torch.randn(B, H, T, D, generator=g).bfloat16() for _ in range(3))
    inv_temp = D ** -0.5
    res = ops.attn_fwd(q.cuda(), k.cuda(), v.cuda(), inv_temp, no_grad=True, return_attention=True)
    w = res[4]
    assert w.shape == (B, H, T, T)
    for b in range(B):
        _, _, att, _ = orc.sb_dense_fwd(q[b].float().numpy(), k[b].float().numpy(), v[b].float().numpy(), inv_temp,
                                        False, np.float64, return_att=True)
        assert np.abs(w[b].double().cpu().numpy() - att).max() <= TOL_F32


def test_weights_single_sequence_layout():
    """One sequence in the pack: the layout the reference writes ([H, T, T], row = query, column = key)."""
    from stickbreaking_attention_b200 import ops
    H, T, D = 2, 50, 32
    q, k, _, _, _ = synth(H, T, D, 2)
    w = ops.attention_weights(to_dev(q, torch.float32), to_dev(k, torch.float32),
                              torch.tensor([T], dtype=torch.int32, device="cuda"))
    wn = w.cpu().numpy()
    assert np.all(np.triu(wn) == 0)  # nothing on or above the diagonal
    assert np.all(wn.sum(-1) <= 1 + 1e-6)
