"""NystromConfig: defaults and assertion messages of the reference's dataclass
(flash_nystrom/nystrom_config.py:7-93)."""
import math

import pytest

from flashnystrom_b200 import NystromConfig


def test_defaults():
    c = NystromConfig()
    assert (c.num_landmarks, c.newton_iter, c.conv_kernel_size) == (64, 6, 3)
    assert c.use_conv_residual and c.fast_dk2inv and not c.use_tc_pinv
    assert c.kappa_star == 0.0


@pytest.mark.parametrize("kwargs,msg", [
    (dict(num_landmarks=0), "num_landmarks must be positive"),
    (dict(newton_iter=0), "newton_iter must be positive"),
    (dict(conv_kernel_size=-1), "non-negative"),
    (dict(conv_kernel_size=4), "must be odd"),
    (dict(kappa_star=-1.0), "kappa_star"),
    (dict(kappa_star=math.inf), "kappa_star"),
    (dict(kappa_star=math.nan), "kappa_star"),
])
def test_asserts(kwargs, msg):
    with pytest.raises(AssertionError, match=msg):
        NystromConfig(**kwargs)


def test_valid_variants():
    NystromConfig(conv_kernel_size=0)
    NystromConfig(num_landmarks=128, newton_iter=8, kappa_star=5.0, conv_kernel_size=5)
