"""The layer oracle (gated-delta-net step, SiLU) against the reference's C code and its
known answer."""
import numpy as np

from oracle import qwen35_layers_oracle as lo


def test_gdn_step_known_answer_of_the_reference_test():
    # test/test_fortai_smoke.f90:268-282
    state = np.array([[1, 2], [3, 4]], np.float32)
    out = lo.gdn_step(state, np.array([1, 2], np.float32), np.array([5, 6], np.float32),
                      np.array([2, 1], np.float32), 0.5, 0.25, 1.0 / np.sqrt(np.float32(2.0)))
    assert np.abs(out - np.array([4.5, 5.5], np.float32) / np.sqrt(np.float32(2.0))).max() < 1e-5
    assert np.abs(state.reshape(-1) - np.array([1.125, 2.25, 1.625, 2.25], np.float32)).max() < 1e-5


def test_gdn_step_and_silu_match_the_compiled_reference(reference):
    rng = np.random.default_rng(3)
    for hs in (2, 16, 128):
        state = rng.standard_normal((hs, hs)).astype(np.float32)
        key = rng.standard_normal(hs).astype(np.float32) / np.float32(np.sqrt(hs))
        value = rng.standard_normal(hs).astype(np.float32)
        query = rng.standard_normal(hs).astype(np.float32) / np.float32(np.sqrt(hs))
        mine_state, ref_state = state.copy(), state.copy()
        mine = lo.gdn_step(mine_state, key, value, query, 0.9, 0.3, 1.0 / np.sqrt(np.float32(hs)))
        theirs = reference.gdn_step(ref_state, key, value, query, 0.9, 0.3,
                                    float(1.0 / np.sqrt(np.float32(hs))))
        # the reference's AVX2 path sums eight lanes at a time: same values, other order
        assert np.abs(mine - theirs).max() <= 1e-5 * max(1.0, float(np.abs(theirs).max()))
        assert np.abs(mine_state - ref_state).max() <= 1e-5 * float(np.abs(ref_state).max())
    x = np.linspace(-19, 19, 777).astype(np.float32)
    assert np.abs(lo.silu(x) - reference.silu(x)).max() <= 2e-5
