"""The torch.library registration: fake (meta) propagation on CPU, real kernel on the GPU."""
import pytest
import torch

from gemm_b200 import torch_ops  # noqa: F401  (registers torch.ops.neogemm.*)


def test_fake_implementation_gives_shapes_without_a_gpu():
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        x = torch.empty(3, 5, 256, dtype=torch.bfloat16)
        w = torch.empty(136, 256, dtype=torch.bfloat16)
        y = torch.ops.neogemm.linear(x, w)
        assert y.shape == (3, 5, 136) and y.dtype == torch.bfloat16
        out = torch.empty(3, 5, 136, dtype=torch.bfloat16)
        assert torch.ops.neogemm.linear_out(x, w, out) is None


def test_bad_arguments_are_rejected():
    x = torch.empty(4, 32, dtype=torch.bfloat16)
    with pytest.raises(Exception):
        torch.ops.neogemm.linear(x, torch.empty(8, 16, dtype=torch.bfloat16))
    with pytest.raises(Exception):
        torch.ops.neogemm.linear(x.float(), torch.empty(8, 32, dtype=torch.float32))
    with pytest.raises(Exception):   # CPU tensors: there is no CPU implementation
        torch.ops.neogemm.linear(x, torch.empty(8, 32, dtype=torch.bfloat16))


@pytest.mark.gpu
def test_custom_op_and_module_on_the_gpu():
    from gemm_b200.inputs import make_problem
    from oracle import oracle
    A, W = make_problem(40, 1024, 512, seed=12)
    x = A.view(5, 8, 512).cuda()
    y = torch.ops.neogemm.linear(x, W.cuda())
    assert y.shape == (5, 8, 1024)
    oracle.assert_parity(y.reshape(40, 1024), oracle.gemm_fp32(A, W), "torch.ops.neogemm.linear")
    out = torch.full((5, 8, 1024), float("nan"), dtype=torch.bfloat16, device="cuda")
    torch.ops.neogemm.linear_out(x, W.cuda(), out)
    assert torch.equal(out.view(torch.int16), y.view(torch.int16))
    layer = torch_ops.NeoLinear(512, 1024, device="cuda")
    z = layer(x)
    oracle.assert_parity(z.reshape(40, 1024), oracle.gemm_fp32(A, layer.weight.detach().cpu()),
                         "NeoLinear")
