"""torch.ops.afb.bf16_aintb_gemm: the PyTorch operator over the C ABI (awesome_fusion_b200/torch_op.py).
CPU: registration, shape inference, argument checks, and that there is no CPU implementation.
GPU: the operator against the oracle, and a CUDA-graph replay against a direct call."""
import numpy as np
import pytest
import torch

import afb_testlib as T


def _tensors(case, device):
    a = torch.from_numpy(case.a.view(np.int16)).view(torch.bfloat16).to(device)
    b = torch.from_numpy(case.b.view(np.int8) if case.bits == 8 else case.b).to(device)
    if case.scale_dtype == 1:
        s = torch.from_numpy(case.scale.view(np.int16)).view(torch.bfloat16).to(device)
    else:
        s = torch.from_numpy(case.scale).to(device)
    return a, b, s


def test_operator_is_registered_and_infers_shapes():
    import awesome_fusion_b200.torch_op  # noqa: F401  (registers the operator)
    op = torch.ops.afb.bf16_aintb_gemm
    a = torch.empty((4, 256), dtype=torch.bfloat16, device="meta")
    b8 = torch.empty((64, 256), dtype=torch.int8, device="meta")
    b4 = torch.empty((64, 128), dtype=torch.uint8, device="meta")
    out = op(a, b8, torch.empty((64,), dtype=torch.float32, device="meta"), 8, 0, False)
    assert out.shape == (4, 64) and out.dtype == torch.bfloat16
    out = op(a, b4, torch.empty((64, 2), dtype=torch.bfloat16, device="meta"), 4, 128, False)
    assert out.shape == (4, 64)
    with pytest.raises(Exception):   # K of a and b disagree
        op(a, b4, torch.empty((64,), dtype=torch.float32, device="meta"), 8, 0, False)
    with pytest.raises(Exception):   # wrong number of group scales
        op(a, b4, torch.empty((64, 3), dtype=torch.bfloat16, device="meta"), 4, 128, False)


def test_operator_has_no_cpu_path():
    import awesome_fusion_b200.torch_op  # noqa: F401
    a = torch.zeros((1, 64), dtype=torch.bfloat16)
    b = torch.zeros((8, 64), dtype=torch.int8)
    s = torch.ones((8,), dtype=torch.float32)
    with pytest.raises(Exception):
        torch.ops.afb.bf16_aintb_gemm(a, b, s, 8, 0, False)


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k,bits,group,enc", [(4, 512, 1024, 8, 0, 0), (16, 256, 2048, 4, 128, 0), (200, 384, 512, 8, 0, 1), (320, 256, 1024, 4, 128, 1)])
def test_operator_matches_oracle(oracle, m, n, k, bits, group, enc):
    import awesome_fusion_b200.torch_op  # noqa: F401
    case = T.make_case(m, n, k, bits=bits, group=group, enc=enc, seed=71)
    # group-scaled prefill feeds bf16_rn(q * s) to the tensor cores: compared with the oracle given the same rounded weights
    ref = oracle.gemm(case, threads=4, round_w=bool(group and m > 16))
    a, b, s = _tensors(case, "cuda")
    out = torch.ops.afb.bf16_aintb_gemm(a, b, s, bits, group, enc == 1)
    torch.cuda.synchronize()
    got = out.view(torch.int16).cpu().numpy().view(np.uint16)
    mx, nrms, _ = oracle.compare(ref, got, T.rms(ref) * 0.05)
    assert mx <= 1e-2 and nrms < 3e-3, (mx, nrms)


@pytest.mark.gpu
def test_decode_graph_replay_equals_direct_call():
    from awesome_fusion_b200 import torch_op
    case = T.make_case(8, 1024, 2048, bits=4, group=128, seed=72)
    a, b, s = _tensors(case, "cuda")
    direct = torch.ops.afb.bf16_aintb_gemm(a, b, s, 4, 128, False)
    g = torch_op.DecodeGraph(a, b, s, bits=4, group_size=128)
    first = g.replay().clone()
    a2 = torch.from_numpy(T.make_case(8, 1024, 2048, bits=4, group=128, seed=73).a.view(np.int16)).view(torch.bfloat16).cuda()
    g.a.copy_(a2)                      # new activations into the graph's input buffer
    second = g.replay().clone()
    want2 = torch.ops.afb.bf16_aintb_gemm(a2, b, s, 4, 128, False)
    torch.cuda.synchronize()
    assert torch.equal(first.view(torch.int16), direct.view(torch.int16))
    assert torch.equal(second.view(torch.int16), want2.view(torch.int16))
    # the same with programmatic dependent launch inside the graph (weights declared constant): identical bits
    gp = torch_op.DecodeGraph(a2, b, s, bits=4, group_size=128, weights_constant=True)
    third = gp.replay().clone()
    torch.cuda.synchronize()
    assert torch.equal(third.view(torch.int16), want2.view(torch.int16))
