"""CPU: the numpy oracle against the unmodified reference library, live.

Runs only where oracle/_ref/libdnn_ref.so exists (the container that holds the
reference sources); the committed golden vectors cover the same ground where
it does not."""
import numpy as np
import pytest

from cases import CASES, compare


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.name)
def test_reference_matches_oracle(ref, case):
    rng = np.random.default_rng(1234)
    inp = case.make(rng)
    got = case.run(ref, inp)
    ref.reset_step()
    compare(case, got, case.oracle(inp))
