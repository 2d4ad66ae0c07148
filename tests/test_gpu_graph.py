"""Forward and backward captured into a CUDA graph and replayed on new data: the launchers enqueue kernels on the
caller's stream and nothing else (no host synchronisation, no allocation by the library), so a whole step replays
from one graph launch.  Results must be the bits of the eager call."""
import numpy as np
import pytest
import torch

from util import synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("D,dtype", [(128, torch.bfloat16), (16, torch.float32)])
def test_forward_backward_replay_from_a_cuda_graph(D, dtype, monkeypatch):
    from stickbreaking_attention_b200 import check_status, sb_attn_varlen
    monkeypatch.setenv("SBATTN_CHECK_STATUS", "0")  # the per-call status check synchronises, which a capture forbids
    lengths = [300, 129, 64, 200]
    H, T = 2, sum(lengths)
    cu = torch.tensor(np.cumsum(lengths), dtype=torch.int32, device="cuda")

    def load(seed):
        return [torch.from_numpy(x).to("cuda", dtype) for x in synth(H, T, D, seed)]

    def step(q, k, v, do, dr):
        o, rem = sb_attn_varlen(q, k, v, cu, max(lengths), zero_start=False)
        return (o, rem) + torch.autograd.grad([o, rem], [q, k, v], [do, dr])

    sq, sk, sv, sdo, sdr = load(10)
    for x in (sq, sk, sv):
        x.requires_grad_()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # first calls outside the capture: status word, kernel attributes, allocator pool
        for _ in range(2):
            step(sq, sk, sv, sdo, sdr)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = step(sq, sk, sv, sdo, sdr)
    for seed in (11, 12):
        fresh = load(seed)
        with torch.no_grad():
            for dst, src in zip((sq, sk, sv, sdo, sdr), fresh):
                dst.copy_(src)
        graph.replay()
        torch.cuda.synchronize()
        got = [x.clone() for x in outs]
        q, k, v = (x.clone().requires_grad_() for x in fresh[:3])
        want = step(q, k, v, fresh[3], fresh[4])
        torch.cuda.synchronize()
        for a, b in zip(got, want):
            assert torch.equal(a, b)
    assert check_status() == 0
