"""The CUDA path on the reference's golden vectors for fused linear, fusion, convolution and
contract/expand (tests/golden/families.npz).  Forwards are bit-exact; gradients whose summation
order is free within 1e-5 of the summed term magnitudes (computed by the oracle on the same inputs)."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN, grad_close
from oracle import hinge_oracle as ho

pytestmark = pytest.mark.gpu

FAMILIES = np.load(os.path.join(GOLDEN, "families.npz"))


def case(prefix):
    n = len(prefix)
    return {k[n:]: FAMILIES[k] for k in FAMILIES.files if k.startswith(prefix)}


def dev(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("idx", range(int(FAMILIES["linear_count"])))
def test_fused_linear_and_fusion_golden(idx):
    from hingetreefortorch_b200 import _cabi
    c = case("linear%02d_" % idx)
    kind = str(c["kind"])
    d = {k: dev(v) for k, v in c.items() if k != "kind"}
    vec = d.get("vec")
    fam = _cabi.ForestFamily(kind, d["x"], d["w"], vec=vec, lin=d["lin"])
    out = fam.linear_forward(d["x"], vec, d["thr"], d["ord"], d["w"], d["lin"], d["bias"])
    assert np.array_equal(out.cpu().numpy(), c["out"])
    gx, gvec, gthr, gw, glin = fam.linear_backward(d["x"], vec, d["thr"], d["ord"], d["w"], d["lin"], d["g"])
    mag = ho.magnitudes(ho.linear_backward, kind, c["x"], c["thr"], c["ord"], c["w"], c["lin"], c["g"], vec=c.get("vec"))
    ax, athr, aw, alin = mag[0], mag[-4], mag[-3], mag[-2]
    assert grad_close(gx, c["gx"], ax) and grad_close(gthr, c["gthr"], athr)
    assert grad_close(gw, c["gw"], aw) and grad_close(glin, c["glin"], alin)
    if vec is not None:
        assert grad_close(gvec, c["gvec"], mag[1])
        plain = _cabi.ForestFamily(kind, d["x"], d["w"], vec=vec)
        assert np.array_equal(plain.fusion_forward(d["x"], vec, d["thr"], d["ord"], d["w"]).cpu().numpy(), c["fusion_out"])
        gimg, gvec, gthr, gw = plain.fusion_backward(d["x"], vec, d["thr"], d["ord"], d["w"], d["fusion_g"])
        aimg, avec, athr, aw = ho.magnitudes(ho.backward, kind, c["x"], c["thr"], c["ord"], c["w"], c["fusion_g"], vec=c["vec"])
        assert grad_close(gimg, c["fusion_gx"], aimg) and grad_close(gvec, c["fusion_gvec"], avec)
        assert grad_close(gthr, c["fusion_gthr"], athr) and grad_close(gw, c["fusion_gw"], aw)


@pytest.mark.parametrize("idx", range(int(FAMILIES["conv_count"])))
def test_convolution_golden(idx):
    from hingetreefortorch_b200 import _cabi
    c = case("conv%02d_" % idx)
    kind = str(c["kind"])
    geometry = [tuple(int(v) for v in row) for row in c["geometry"]]
    d = {k: dev(v) for k, v in c.items() if k not in ("kind", "geometry")}
    conv = _cabi.Conv(kind, d["x"], d["w"], *geometry)
    assert np.array_equal(conv.forward(d["x"], d["thr"], d["ord"], d["w"]).cpu().numpy(), c["out"])
    gx, gthr, gw = conv.backward(d["x"], d["thr"], d["ord"], d["w"], d["g"])
    ax, athr, aw = ho.magnitudes(ho.conv_backward, kind, c["x"], c["thr"], c["ord"], c["w"], c["g"], *geometry)
    assert grad_close(gx, c["gx"], ax) and grad_close(gthr, c["gthr"], athr) and grad_close(gw, c["gw"], aw)


@pytest.mark.parametrize("idx", range(int(FAMILIES["patch_count"])))
def test_contract_expand_golden(idx):
    from hingetreefortorch_b200 import _cabi
    c = case("patch%02d_" % idx)
    window, padding = tuple(int(v) for v in c["window"]), tuple(int(v) for v in c["padding"])
    contracted = _cabi.contract(dev(c["x"]), window, padding)
    assert np.array_equal(contracted.cpu().numpy(), c["contracted"])
    assert np.array_equal(_cabi.expand(contracted, padding).cpu().numpy(), c["expanded"])
