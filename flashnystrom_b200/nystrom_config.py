"""Configuration dataclass, field-for-field the reference's NystromConfig
(flash_nystrom/nystrom_config.py:7-93): same names, defaults and assertion messages."""
import math
from dataclasses import dataclass


@dataclass
class NystromConfig:
    num_landmarks: int = 64
    """Number of landmark (inducing) points m."""

    newton_iter: int = 6
    """Newton-Schulz iterations of the pseudoinverse.  The backward differentiates through
    every unrolled iterate, so gradients are exact whatever the convergence."""

    conv_kernel_size: int = 3
    """Kernel size of the depthwise conv1d residual over V; 0 disables it."""

    use_conv_residual: bool = True

    fast_dk2inv: bool = True
    """Accepted for compatibility.  This library always forms dK2inv = dstep2 * Bmat^T from
    the FP32 Bmat saved by the forward, so the flag selects nothing."""

    kappa_star: float = 0.0
    """Tikhonov ridge target condition number: when > 0 the pseudoinverse inverts
    M = K2^T K2 + lambda I with lambda = ||K2||_1 ||K2||_inf / kappa_star (lambda detached)."""

    use_tc_pinv: bool = False
    """Accepted for compatibility.  The pseudoinverse always runs in FP32."""

    def __post_init__(self):
        assert self.num_landmarks > 0, "num_landmarks must be positive"
        assert self.newton_iter > 0, "newton_iter must be positive"
        assert self.conv_kernel_size >= 0, "conv_kernel_size must be non-negative"
        if self.conv_kernel_size > 0:
            assert self.conv_kernel_size % 2 == 1, "conv_kernel_size must be odd"
        assert math.isfinite(self.kappa_star) and self.kappa_star >= 0.0, \
            "kappa_star must be finite and >= 0 (0 disables the Tikhonov ridge)"
