"""``jaxdecomp_b200.fft``: the distributed transforms under the module path the reference uses
(``jaxdecomp.fft.pfft3d`` and friends, ``src/jaxdecomp/fft.py:127-354``).  The implementations live in
:mod:`jaxdecomp_b200.ops.fft`."""
from .ops.fft import fftfreq3d, pfft3d, pifft3d, pirfft3d, prfft3d, rfftfreq3d

__all__ = ["pfft3d", "pifft3d", "prfft3d", "pirfft3d", "fftfreq3d", "rfftfreq3d"]
