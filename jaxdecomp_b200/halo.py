"""``jaxdecomp_b200.halo``: halo exchange under the module path the reference uses
(``jaxdecomp.halo.halo_exchange``, ``src/jaxdecomp/halo.py:8-80``), with the in-place, accumulate and
pad/crop helpers of this library.  The implementations live in :mod:`jaxdecomp_b200.ops.halo`."""
from .ops.halo import halo_accumulate, halo_exchange, halo_exchange_, halo_reduce, pad_halo, unpad_halo

__all__ = ["halo_exchange", "halo_exchange_", "halo_accumulate", "halo_reduce", "pad_halo", "unpad_halo"]
