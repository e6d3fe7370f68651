"""The workload registry: deterministic seeded inputs and the byte accounting that
the roofline figures use."""
import pytest
import torch

from credit_b200 import workloads as W


def test_algorithmic_bytes_of_the_headline_shapes():
    assert W.algorithmic_bytes("rmsnorm_forward", 1024, 32768) == 268_566_528
    assert W.algorithmic_bytes("row_reduce", 512, 1_048_576) == 2_147_491_840
    assert W.algorithmic_bytes("layernorm_forward", 4096, 131072) == 2_148_564_992
    assert W.algorithmic_bytes("layernorm_backward_stats", 8192, 65536) == 3_222_077_440


def test_default_shapes():
    assert (W.WORKLOADS["rmsnorm_forward"].rows, W.WORKLOADS["rmsnorm_forward"].cols) == (1024, 32768)
    assert (W.WORKLOADS["row_reduce"].rows, W.WORKLOADS["row_reduce"].cols) == (512, 1048576)
    assert W.WORKLOADS["layernorm_backward"].reductions_per_stage == (2, 2)
    assert W.WORKLOADS["layernorm_backward"].barrier_count == 2
    assert W.WORKLOADS["layernorm_backward_stats"].partial_count == 2


@pytest.mark.parametrize("name", ["rmsnorm_forward", "row_reduce", "layernorm_forward",
                                  "layernorm_backward_stats"])
def test_factories_are_deterministic(name):
    spec = W.WORKLOADS[name]
    a = spec.input_factory(4, 256, torch.device("cpu"))
    b = spec.input_factory(4, 256, torch.device("cpu"))
    for ta, tb in zip(a, b):
        assert torch.equal(ta, tb)
    assert a[0].shape == (4, 256) and a[0].dtype == spec.dtype
    c = spec.input_factory(4, 256, torch.device("cpu"), seed=1)
    assert not torch.equal(a[0], c[0])


def test_row_reduce_inputs_have_one_planted_maximum():
    (x,) = W.make_row_reduce_inputs(16, 4096, torch.device("cpu"))
    assert torch.all(x.amax(dim=-1) == 10.0)
    assert torch.all((x == 10.0).sum(dim=-1) == 1)


def test_layernorm_backward_stats_inputs_carry_matching_statistics():
    x, dy, gamma, mean, rstd = W.make_layernorm_backward_stats_inputs(8, 512, torch.device("cpu"))
    assert x.dtype == torch.bfloat16 and mean.dtype == torch.float32
    torch.testing.assert_close(mean, x.float().mean(-1))
    torch.testing.assert_close(rstd, torch.rsqrt(x.float().var(-1, unbiased=False) + 1e-5))
    assert float(gamma.min()) >= 0.5 and float(gamma.max()) <= 1.5


def test_reference_style_layernorm_inputs_follow_the_global_seed():
    torch.manual_seed(1234 + 64)
    a = W.make_layernorm_inputs(2, 64, torch.device("cpu"))
    torch.manual_seed(1234 + 64)
    b = W.make_layernorm_inputs(2, 64, torch.device("cpu"))
    assert all(torch.equal(p, q) for p, q in zip(a, b))
    assert float(a[2].min()) >= 0.75 and float(a[2].max()) <= 1.25
