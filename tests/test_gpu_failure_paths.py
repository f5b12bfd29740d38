"""Refusals of the forward pass, injected on the host only: artifacts and adapters whose constants
leave an integer-domain gate (tests/golden/failure_cases.py). Each case is a short script of
sslm_* calls; tests/golden/failure_golden.json holds what the reference's CPU library returned
call by call -- status, tokens consumed or produced, and a digest of what each sequence observably
holds afterwards (header fields, mid-token residual, the K/V of the positions that count). The
CUDA library must return the same, which covers: the first failing site in the reference's
program order (one artifact trips two sites), SSLM_NUMERIC_STEP_REFUSED versus
SSLM_ARTIFACT_REJECTED, a refused call leaving the sequence where the last committed layer left
it, a batch in which the sequences before the refused one have advanced and the ones after it
have not, and recovery once the offending adapter is detached. Where the compiled reference
travels with the tree it is also run live beside the records.
"""
import json
import os

import pytest

import failure_cases as F

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "failure_golden.json")


@pytest.fixture(scope="module")
def golden():
    with open(GOLDEN) as f:
        return json.load(f)


def as_json(rec):
    return json.loads(json.dumps(rec))


@pytest.mark.parametrize("name", sorted(F.ARTIFACTS))
def test_hostile_artifact_is_refused_like_the_reference(gpu_lib, golden, name):
    got = as_json(F.run_artifact_case(gpu_lib, name))
    assert got == golden[name]
    if name in F.BIAS_BITS:
        # the landings the reference's walk had reached stay counted in kv_saturation_count (the only
        # field a refused prefill moves): both refused calls changed the digest
        assert len({r[-1] for r in got[:3]}) == 3
    else:
        # the refusal left nothing behind: every digest equals the fresh sequence's
        assert len({r[-1] for r in got}) == 1


def test_batch_in_which_one_sequence_is_refused(gpu_lib, golden):
    got = as_json(F.run_batch_case(gpu_lib))
    assert got == golden["batch_row3_refused"]
    step = [r for r in got if r[0] == "decode1"][0]
    assert step[1] != 0 and step[3][4] is True and step[3][:3] == [False, False, False]


def test_refusal_in_the_second_layer_of_a_sliced_token(gpu_lib, golden):
    assert as_json(F.run_mid_token_case(gpu_lib)) == golden["mid_token_refused"]


def test_layers_before_a_refused_layer_stay_committed(gpu_lib, golden):
    assert as_json(F.run_partial_commit_case(gpu_lib)) == golden["partial_commit"]


def test_records_still_match_the_live_reference(ref_lib, golden):
    assert as_json(F.run_batch_case(ref_lib)) == golden["batch_row3_refused"]
    assert as_json(F.run_artifact_case(ref_lib, "two_sites")) == golden["two_sites"]
