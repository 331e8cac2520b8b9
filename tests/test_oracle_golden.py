"""Pins the CPU oracle against the reference's own golden vectors."""
import pytest

from . import golden_cases
from .backends import OracleBackend


@pytest.mark.parametrize("case", golden_cases.ALL, ids=lambda f: f.__name__)
def test_oracle_matches_reference_vectors(case, orc):
    case(OracleBackend())


def test_oracle_uses_openblas(orc):
    assert orc.lib().orc_blas_loaded() == 1, "SciPy's bundled OpenBLAS should be found in this image"
