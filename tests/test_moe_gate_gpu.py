"""GPU parity of the MoE router (projection through wuda_gemm_bf16, routing through wuda_moe_route)
against the CPU oracle and the fixture made with the origin's Gate."""
import numpy as np
import pytest
import torch

import oracle
from conftest import load_golden

pytestmark = pytest.mark.gpu


def from_u16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).cuda()


@pytest.mark.parametrize("name", ["softmax", "sigmoid", "sqrtsoftplus"])
def test_golden_gate(wuda, name):
    g = load_golden("moe_gate_256.npz")
    logits = torch.empty(g["x"].shape[0], g["weight"].shape[0], dtype=torch.float32, device="cuda")
    w, idx = wuda.moe_gate(from_u16(g["x"]), from_u16(g["weight"]), torch.from_numpy(g["bias"]).cuda(), name,
                           float(g["route_scale"]), int(g["topk"]), logits=logits)
    torch.cuda.synchronize()
    assert np.array_equal(idx.cpu().numpy(), g["indices_" + name])
    assert np.abs(w.cpu().numpy() - g["weights_" + name]).max() <= 2e-6
    # the router alone, on the GPU's own logits: the same experts as the oracle, weights to rounding
    code = {"softmax": 0, "sigmoid": 1, "sqrtsoftplus": 2}[name]
    ow, oi = oracle.moe_route(logits.cpu().numpy(), g["bias"], int(g["topk"]), code, float(g["route_scale"]))
    assert np.array_equal(idx.cpu().numpy(), oi)
    assert np.abs(w.cpu().numpy() - ow).max() <= 1e-6


@pytest.mark.parametrize("tokens,experts,k,code", [(1, 256, 8, 2), (64, 256, 8, 2), (130, 256, 8, 1), (9, 40, 5, 0),
                                                   (33, 512, 32, 2), (5, 8, 8, 1)])
def test_router_against_oracle(wuda, tokens, experts, k, code):
    from wuda_b200._lib import check
    rng = np.random.default_rng(tokens + experts)
    logits = rng.normal(size=(tokens, experts)).astype(np.float32) * 2
    logits[0, : min(6, experts)] = 1.25                       # exact ties: the lower expert first
    bias = (rng.normal(size=experts) * 0.1).astype(np.float32)
    w = torch.empty(tokens, k, device="cuda")
    idx = torch.empty(tokens, k, dtype=torch.int32, device="cuda")
    lg, b = torch.from_numpy(logits).cuda(), torch.from_numpy(bias).cuda()
    check(wuda.lib.wuda_moe_route(lg.data_ptr(), b.data_ptr(), w.data_ptr(), idx.data_ptr(), tokens, experts, k, code,
                                  1.5, None))
    torch.cuda.synchronize()
    ow, oi = oracle.moe_route(logits, bias, k, code, 1.5)
    assert np.array_equal(idx.cpu().numpy(), oi)
    assert np.abs(w.cpu().numpy() - ow).max() <= 2e-6


def test_rejects_bad_arguments(wuda):
    from wuda_b200._lib import check
    lg = torch.zeros(2, 16, device="cuda")
    w, idx = torch.empty(2, 4, device="cuda"), torch.empty(2, 4, dtype=torch.int32, device="cuda")
    with pytest.raises(wuda.WudaError, match="k must be"):
        check(wuda.lib.wuda_moe_route(lg.data_ptr(), None, w.data_ptr(), idx.data_ptr(), 2, 16, 17, 1, 1.0, None))
    with pytest.raises(wuda.WudaError, match="score_func"):
        check(wuda.lib.wuda_moe_route(lg.data_ptr(), None, w.data_ptr(), idx.data_ptr(), 2, 16, 4, 3, 1.0, None))
