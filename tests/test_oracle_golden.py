"""The CPU restatement (oracle/small_oracle.c) against the reference's own golden vectors
(PyTorch-generated, test/regression_data of the reference; copies under tests/golden).
Tolerance is the reference tests' own almost_equal (rtol 5e-3, atol 1e-5,
test/test_utils.hpp:41-46); max pooling is compared exactly as test/test_maxpool.cpp:101
does.  Each case runs with the REF blocking (1) and the B200 blocking (16)."""
import numpy as np
import pytest

from oracle.bindings import shape
from smallframework_b200 import packing as P
from tests.util import case_id, case_pads, golden_cases, read_bin, reference_close

BLOCKS = (1, 16)


def _cases(kind):
    cs = golden_cases(kind)
    assert cs, f"no golden cases of kind {kind}"
    return [pytest.param(c, id=case_id(c)) for c in cs]


@pytest.mark.parametrize("cb", BLOCKS)
@pytest.mark.parametrize("c", _cases("conv2d"))
def test_conv2d(oracle, c, cb):
    x = read_bin(c["x"]).reshape(c["C"], c["H"], c["W"])
    w = read_bin(c["w"]).reshape(c["K"], c["C"], c["k"], c["k"])
    s = shape(c["C"], c["K"], c["H"], c["W"], c["k"], c["k"], c["s"], case_pads(c), cb)
    ho, wo = s.out_hw()
    y = read_bin(c["y"]).reshape(c["K"], ho, wo)
    got = oracle.conv2d_f32(s, P.pack_activation(x, cb), P.pack_conv_filter(w, cb, cb))
    assert reference_close(P.unpack_activation(got, c["K"], ho, wo, cb), y)


@pytest.mark.parametrize("cb", BLOCKS)
@pytest.mark.parametrize("c", _cases("dw_conv"))
def test_dw_conv(oracle, c, cb):
    x = read_bin(c["x"]).reshape(c["C"], c["H"], c["W"])
    w = read_bin(c["w"]).reshape(c["C"], c["k"], c["k"])
    s = shape(c["C"], c["C"], c["H"], c["W"], c["k"], c["k"], c["s"], case_pads(c), cb)
    ho, wo = s.out_hw()
    y = read_bin(c["y"]).reshape(c["C"], ho, wo)
    got = oracle.conv2d_f32(s, P.pack_activation(x, cb), P.pack_dw_filter(w, cb), depthwise=True)
    assert reference_close(P.unpack_activation(got, c["C"], ho, wo, cb), y)


@pytest.mark.parametrize("cb", BLOCKS)
@pytest.mark.parametrize("c", _cases("maxpool"))
def test_maxpool(oracle, c, cb):
    x = read_bin(c["x"]).reshape(c["C"], c["H"], c["W"])
    s = shape(c["C"], c["C"], c["H"], c["W"], c["k"], c["k"], c["s"], case_pads(c), cb)
    ho, wo = s.out_hw()
    y = read_bin(c["y"]).reshape(c["C"], ho, wo)
    got = oracle.pool2d_f32(s, P.pack_activation(x, cb))
    assert np.array_equal(P.unpack_activation(got, c["C"], ho, wo, cb), y)


@pytest.mark.parametrize("cb", BLOCKS)
@pytest.mark.parametrize("c", _cases("averagepool"))
def test_averagepool(oracle, c, cb):
    x = read_bin(c["x"]).reshape(c["C"], c["H"], c["W"])
    s = shape(c["C"], c["C"], c["H"], c["W"], c["k"], c["k"], c["s"], case_pads(c), cb)
    ho, wo = s.out_hw()
    y = read_bin(c["y"]).reshape(c["C"], ho, wo)
    got = oracle.pool2d_f32(s, P.pack_activation(x, cb), average=True)
    assert reference_close(P.unpack_activation(got, c["C"], ho, wo, cb), y)


@pytest.mark.parametrize("c", _cases("relu"))
def test_relu(oracle, c):
    x = read_bin(c["x"]); y = read_bin(c["y"])
    assert np.array_equal(oracle.relu_f32(x), y)


@pytest.mark.parametrize("cb", BLOCKS)
@pytest.mark.parametrize("c", _cases("softmax"))
def test_softmax(oracle, c, cb):
    x = read_bin(c["x"]).reshape(c["C"], c["H"], c["W"])
    y = read_bin(c["y"]).reshape(c["C"], c["H"], c["W"])
    got = oracle.softmax_f32(c["C"], c["H"], c["W"], cb, P.pack_activation(x, cb))
    assert reference_close(P.unpack_activation(got, c["C"], c["H"], c["W"], cb), y)


@pytest.mark.parametrize("cb", BLOCKS)
@pytest.mark.parametrize("c", _cases("partial_bias"))
def test_partial_bias(oracle, c, cb):
    # test/test_partial_bias.cpp:172-194: bias[c] = c accumulated onto the pool input
    x = read_bin(c["x"]).reshape(c["C"], c["H"], c["W"])
    y = read_bin(c["y"]).reshape(c["C"], c["H"], c["W"])
    bias = np.arange(c["C"], dtype=np.float32)
    got = oracle.bias_f32(c["C"], c["H"], c["W"], cb, bias, out=P.pack_activation(x, cb))
    assert reference_close(P.unpack_activation(got, c["C"], c["H"], c["W"], cb), y)
