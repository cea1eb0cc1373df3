"""Pins the CPU oracle against the reference's recorded MLX vectors (no GPU needed)."""
import pytest

import golden_cases
from replay import OracleBackend, check_case

CASES = golden_cases.cases()


@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
def test_oracle_matches_recording(case):
    check_case(case, OracleBackend())
