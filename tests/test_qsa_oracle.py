"""The CPU restatement of query-sparse paged attention (oracle/qsa.py) against the committed outputs of
the reference's own kernels (tests/golden/qsa_ref_sm100a.npz, made by tests/golden/make_golden_qsa.py
on a B200): TQ4 and FP8 E4M3 pools, without gate, with the sigmoid gate, with gate + Hadamard-64."""
import os

import numpy as np
import pytest

FIXTURE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "qsa_ref_sm100a.npz")


@pytest.fixture(scope="module")
def fx(oracle_lib):
    if not os.path.exists(FIXTURE):
        pytest.skip("fixture not generated yet")
    return dict(np.load(FIXTURE))


def _f16(bits):
    return bits.view(np.float16).astype(np.float32)


@pytest.mark.parametrize("fmt_name", ["tq4", "fp8"])
@pytest.mark.parametrize("variant", ["plain", "gated", "hadamard"])
def test_restatement_matches_the_reference_kernels(fx, fmt_name, variant):
    from oracle import qsa
    fmt = qsa.TQ4 if fmt_name == "tq4" else qsa.FP8_E4M3
    q, gate = _f16(fx["q"]), _f16(fx["gate"])
    T, hq = q.shape[0], q.shape[1]
    hkv = fx[f"{fmt_name}_k_pool"].shape[1]
    got = qsa.sparse_attention(fx[f"{fmt_name}_k_pool"], fx[f"{fmt_name}_v_pool"], fmt, fmt, q,
                               None if variant == "plain" else gate, fx["sel_phys"], fx["sel_logical"],
                               fx["num_selected"], fx["seq_pos"], fx["valid_token_mask"], hq, hkv, 0.0625,
                               variant == "hadamard")
    want_bits = fx[f"{fmt_name}_out_{variant}"]
    want = _f16(want_bits)
    # masked token and the token without entries: exact zeros in the reference's output
    assert (want_bits[3] == 0).all() and (want[2] == 0).all()
    assert np.abs(want[[0, 1, 4]]).max() > 0.05
    # fp32 kernels against float64: a few fp16 steps (the kernels exponentiate with the fast variants)
    assert np.all(np.abs(got - want) <= 1e-3 + 4e-3 * np.abs(want)), float(np.abs(got - want).max())


def test_fixture_holds_the_edge_cases(fx):
    assert (fx["sel_phys"][0] < 0).any() and fx["num_selected"][2] == 0 and fx["valid_token_mask"][3] == 0
    own = fx["seq_pos"] // 4
    assert all(own[t] in fx["sel_logical"][t, :fx["num_selected"][t]] for t in (0, 1, 4))
    beyond = [(fx["sel_logical"][t, :fx["num_selected"][t]] * 4 > fx["seq_pos"][t]).any() for t in range(5)]
    assert any(beyond)
