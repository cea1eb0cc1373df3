"""The CUDA path against the reference's recorded MLX vectors (through the C ABI)."""
import pytest

import golden_cases
from replay import check_case

pytestmark = pytest.mark.gpu
CASES = golden_cases.cases()


@pytest.fixture(scope="module")
def backend():
    from cuda_backend import CudaBackend
    return CudaBackend()


@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
def test_cuda_matches_recording(case, backend):
    check_case(case, backend)
