"""The oracle and the product's host-side tables against tables dumped from the reference's own Python code."""

import numpy as np
import pytest
import torch

from lunaequivariance_b200.coupling import cg_terms, wigner_3j
from lunaequivariance_b200.irreps import Irrep, Irreps
from lunaequivariance_b200.paths import TensorProductPaths, build_uvu_conv_metadata
from oracle import uvu_conv as oracle_conv


def test_wigner_matches_reference(golden_npz):
    data = golden_npz("reference_wigner.npz")
    assert len(data.files) > 60
    for key in data.files:
        l1, l2, l3 = (int(v) for v in key.split("_"))
        np.testing.assert_allclose(wigner_3j(l1, l2, l3), data[key], atol=1e-14, rtol=0)
        np.testing.assert_allclose(oracle_conv.real_cg(l1, l2, l3), data[key], atol=1e-13, rtol=0)


def test_wigner_is_unit_norm_and_rejects_bad_triples():
    assert abs(np.sum(wigner_3j(2, 3, 3) ** 2) - 1.0) < 1e-14
    with pytest.raises(ValueError):
        wigner_3j(0, 1, 3)


def _paths(entry):
    return TensorProductPaths(
        entry["irreps_in1"], entry["irreps_in2"], entry["irreps_out"],
        [tuple(i) for i in entry["instructions_in"]],
        internal_weights=False, shared_weights=False, **entry["kwargs"],
    )


def test_path_normalisation_matches_reference(reference_tables):
    for name, entry in reference_tables.items():
        paths = _paths(entry)
        assert paths.weight_numel == entry["weight_numel"], name
        assert len(paths.instructions) == len(entry["instructions"])
        for ours, ref in zip(paths.instructions, entry["instructions"]):
            assert [ours.i_in1, ours.i_in2, ours.i_out, ours.connection_mode, ours.has_weight] == ref[:5]
            assert ours.path_weight == pytest.approx(ref[5], rel=1e-15, abs=0)
            assert list(ours.path_shape) == ref[6]


def test_uvu_metadata_matches_reference(reference_tables):
    for name, entry in reference_tables.items():
        meta = build_uvu_conv_metadata(_paths(entry), torch.float64)
        ref = entry["meta"]
        for key in ("in1_dim", "in2_dim", "out_dim", "weight_numel", "max_channels"):
            assert meta[key] == ref[key], (name, key)
        assert len(meta["generated_specs"]) == len(ref["generated_specs"])
        for ours, theirs in zip(meta["generated_specs"], ref["generated_specs"]):
            for key, value in theirs.items():
                if key == "terms":
                    continue
                assert ours[key] == value, (name, key)
            assert [t[:3] for t in ours["terms"]] == [tuple(t[:3]) for t in theirs["terms"]], name
            np.testing.assert_allclose([t[3] for t in ours["terms"]], [t[3] for t in theirs["terms"]],
                                       atol=1e-14, rtol=0)


def test_oracle_specs_match_reference(reference_tables):
    for name, entry in reference_tables.items():
        meta = oracle_conv.build_specs(entry["irreps_in1"], entry["irreps_in2"], entry["irreps_out"],
                                       [tuple(i) for i in entry["instructions_in"]], **entry["kwargs"])
        ref = entry["meta"]
        assert meta["weight_numel"] == ref["weight_numel"]
        assert (meta["in1_dim"], meta["in2_dim"], meta["out_dim"]) == (ref["in1_dim"], ref["in2_dim"], ref["out_dim"])
        for ours, theirs in zip(meta["specs"], ref["generated_specs"]):
            for key in ("x_offset", "y_offset", "out_offset", "weight_offset", "channels", "d1", "d2", "d3"):
                assert ours[key] == theirs[key], (name, key)
            assert ours["weight_stride"] == theirs.get("weight_stride", 1)
            dense = np.zeros_like(ours["cg"])
            for i, j, k, c in theirs["terms"]:
                dense[i, j, k] = c
            np.testing.assert_allclose(ours["cg"], dense, atol=2e-12, rtol=0)


def test_float32_metadata_narrows_coefficients(reference_tables):
    meta32 = build_uvu_conv_metadata(_paths(reference_tables["small"]), torch.float32)
    meta64 = build_uvu_conv_metadata(_paths(reference_tables["small"]), torch.float64)
    a = [t[3] for s in meta32["generated_specs"] for t in s["terms"]]
    b = [t[3] for s in meta64["generated_specs"] for t in s["terms"]]
    assert len(a) == len(b)
    np.testing.assert_allclose(a, b, rtol=1e-6)


def test_irreps_behaviour():
    irreps = Irreps("32x0e + 32x1o+2e")
    assert str(irreps) == "32x0e+32x1o+1x2e"
    assert irreps.dim == 32 + 96 + 5 and irreps.lmax == 2 and irreps.num_irreps == 65
    assert [s.start for s in irreps.slices()] == [0, 32, 128]
    assert Irrep.parse("1o") in irreps and Irrep.parse("1e") not in irreps
    assert list(Irrep.parse("1o") * Irrep.parse("2e")) == [Irrep(1, -1), Irrep(2, -1), Irrep(3, -1)]
    assert str(Irreps.spherical_harmonics(3)) == "1x0e+1x1o+1x2e+1x3o"
    assert str(Irreps("2x1o+3x1o+0x2e").simplify()) == "5x1o"
    with pytest.raises(ValueError):
        Irreps("3x1q")
    assert cg_terms(1, 1, 0, 1.0)[0][3] == pytest.approx(3 ** -0.5)


def test_metadata_validation_errors(reference_tables):
    with pytest.raises(ValueError, match="equal input/output multiplicities"):
        build_uvu_conv_metadata(TensorProductPaths("3x0e", "1x0e", "2x0e", [(0, 0, 0, "uvu", True)],
                                                   internal_weights=False, shared_weights=False))
    with pytest.raises(ValueError, match="shared_weights=False"):
        build_uvu_conv_metadata(TensorProductPaths("3x0e", "1x0e", "3x0e", [(0, 0, 0, "uvu", True)],
                                                   internal_weights=False, shared_weights=True))
    with pytest.raises(ValueError, match="Only connection_mode='uvu'"):
        build_uvu_conv_metadata(TensorProductPaths("3x0e", "3x0e", "3x0e", [(0, 0, 0, "uuu", True)],
                                                   internal_weights=False, shared_weights=False))
