"""Every catalogued operator, every default case: construct, draw, run on the device, judge.

The shape of iron/tests/operators/test_catalog.py:54-73: seeded vectors (seed 42, scale 4),
the standalone call ``op(*tensors)``, and ``op.judge`` against ``op.reference()`` under
``op.tolerance()``.
"""

import pytest

from iron_b200.operators import CATALOG
from iron_b200.testing import run_test

pytestmark = pytest.mark.gpu

CASES = [(cls, case) for cls in CATALOG for case in cls.test.resolve(cls) if not case.extensive]


@pytest.mark.parametrize("cls,case", CASES, ids=[f"{c.__name__}-{k.label}" for c, k in CASES])
def test_catalogued_case(cls, case):
    result = run_test(cls, case, time=case.bench)
    if cls(**case.kwargs).tolerance() is not None:
        assert result["verdicts"] and all(result["verdicts"].values())
