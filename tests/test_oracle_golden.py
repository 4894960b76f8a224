"""Pins the oracle: both legs must reproduce the outputs the unmodified
reference produced on CPU (tests/golden/reference_cpu_outputs.npz)."""
import pytest
import torch

import oracle
from cases import EAGER_CASES, FUSED_CASES


@pytest.mark.parametrize("idx", range(len(FUSED_CASES)))
def test_fused_cases_match_reference_outputs(golden, idx):
    ishape, wshape, stride, padding, dilation = FUSED_CASES[idx]
    key = f"fused_{idx:02d}"
    x, w, b = (torch.from_numpy(golden[key + s]) for s in ("_x", "_w", "_b"))
    ref = torch.from_numpy(golden[key + "_y"])
    assert tuple(x.shape) == ishape and tuple(w.shape) == wshape
    got_torch = oracle.conv2d_torch_cpu(x, w, b, stride, padding, dilation, 1, relu=True)
    got_loops = oracle.conv2d_loops(x, w, b, stride, padding, dilation, 1, relu=True)
    torch.testing.assert_close(got_torch, ref, rtol=0, atol=0)  # same torch call the reference makes
    torch.testing.assert_close(got_loops, ref, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("idx", range(len(EAGER_CASES)))
def test_eager_cases_match_reference_outputs(golden, idx):
    ishape, wshape, has_bias, stride, padding, dilation, groups = EAGER_CASES[idx]
    key = f"eager_{idx:02d}"
    x, w = torch.from_numpy(golden[key + "_x"]), torch.from_numpy(golden[key + "_w"])
    b = torch.from_numpy(golden[key + "_b"]) if has_bias else None
    ref = torch.from_numpy(golden[key + "_y"])
    got_torch = oracle.conv2d_torch_cpu(x, w, b, stride, padding, dilation, groups)
    got_loops = oracle.conv2d_loops(x, w, b, stride, padding, dilation, groups)
    torch.testing.assert_close(got_torch, ref, rtol=0, atol=0)
    torch.testing.assert_close(got_loops, ref, rtol=2e-5, atol=2e-5)


N_TAIL, N_GELU, N_MM = 3, 2, 5   # cases in tests/golden/make_golden.py::_write_next_rows


@pytest.mark.parametrize("idx", range(N_TAIL))
def test_block_tail_cases_match_reference_outputs(golden_next, idx):
    """relu(conv * scale + bias + shortcut): the oracle's sequence is the reference graph's (conv2d, mul, bias_add, add, relu)."""
    key = f"tail_{idx:02d}"
    x, w, s, b, r, ref = (torch.from_numpy(golden_next[f"{key}_{n}"]) for n in ("x", "w", "s", "b", "r", "y"))
    stride, padding = (int(v) for v in golden_next[key + "_meta"])
    got = torch.relu(oracle.conv2d_torch_cpu(x, w, b, stride, padding, 1, 1, scale=s.reshape(-1)) + r)
    torch.testing.assert_close(got, ref, rtol=0, atol=0)
    loops = torch.relu(oracle.conv2d_loops(x, w, b, stride, padding, 1, 1, scale=s.reshape(-1)) + r)
    torch.testing.assert_close(loops, ref, rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("idx", range(N_GELU))
def test_gelu_cases_match_reference_outputs(golden_next, idx):
    key = f"gelu_{idx:02d}"
    x, w, b, ref = (torch.from_numpy(golden_next[f"{key}_{n}"]) for n in ("x", "w", "b", "y"))
    stride, padding, tanh = (int(v) for v in golden_next[key + "_meta"])
    got = torch.nn.functional.gelu(oracle.conv2d_torch_cpu(x, w, b, stride, padding, 1, 1),
                                   approximate="tanh" if tanh else "none")
    torch.testing.assert_close(got, ref, rtol=0, atol=0)


@pytest.mark.parametrize("idx", range(N_MM))
def test_mm_cases_match_reference_outputs(golden_next, idx):
    """mm as the oracle sees it: a 1x1 convolution over a row of M pixels equals the reference's torch.mm."""
    key = f"mm_{idx:02d}"
    a, b, ref = (torch.from_numpy(golden_next[f"{key}_{n}"]) for n in ("a", "b", "y"))
    torch.testing.assert_close(torch.mm(a, b), ref, rtol=0, atol=0)
    x4 = a.t().unsqueeze(0).unsqueeze(2)                      # [1, K, 1, M]
    w4 = b.t().unsqueeze(-1).unsqueeze(-1)                    # [N, K, 1, 1]
    as_conv = oracle.conv2d_loops(x4.contiguous(), w4.contiguous(), None, 1, 0, 1, 1)[0, :, 0, :].t()
    torch.testing.assert_close(as_conv, ref, rtol=2e-5, atol=2e-5)


def test_loops_double_matches_torch_double():
    g = torch.Generator().manual_seed(7)
    x = torch.randn(2, 6, 11, 9, generator=g, dtype=torch.float64)
    w = torch.randn(4, 3, 3, 2, generator=g, dtype=torch.float64)
    b = torch.randn(4, generator=g, dtype=torch.float64)
    s = torch.rand(4, generator=g, dtype=torch.float64) + 0.5
    a = oracle.conv2d_torch_cpu(x, w, b, (2, 1), (1, 0), (1, 2), 2, scale=s, relu=True, compute_dtype=torch.float64)
    c = oracle.conv2d_loops(x, w, b, (2, 1), (1, 0), (1, 2), 2, scale=s, relu=True, double=True)
    torch.testing.assert_close(a, c, rtol=1e-12, atol=1e-12)


def test_output_size_and_padding_rules():
    assert oracle.conv_out_dim(224, 3, 3, 1, 7, 2) == 112
    assert oracle.conv_out_dim(2, 0, 0, 1, 5, 1) == -2
    assert oracle.normalize_padding((4, 2, 3, 3), (1, 1), "same", (2, 2)) == (2, 2, 2, 2)
    assert oracle.normalize_padding((4, 2, 4, 2), (1, 1), "same", (1, 1)) == (1, 2, 0, 1)
    with pytest.raises(RuntimeError):
        oracle.normalize_padding((4, 2, 3, 3), (2, 2), "same", (1, 1))
