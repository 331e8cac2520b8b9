"""The reference's golden vectors replayed through the C ABI on the GPU."""
import pytest

from . import golden_cases
from .backends import GpuBackend

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", golden_cases.ALL, ids=lambda f: f.__name__)
def test_gpu_matches_reference_vectors(case, gpu):
    case(GpuBackend(gpu))
