"""``jaxdecomp_b200.transpose``: the six pencil transposes under the module path the reference uses
(``jaxdecomp.transpose.transposeXtoY`` and friends, ``src/jaxdecomp/transpose.py:7-242``).  The
implementations live in :mod:`jaxdecomp_b200.ops.transpose`."""
from .ops.transpose import (
    transpose,
    transpose_shard,
    transposeXtoY,
    transposeXtoZ,
    transposeYtoX,
    transposeYtoZ,
    transposeZtoX,
    transposeZtoY,
)

__all__ = ["transpose", "transpose_shard", "transposeXtoY", "transposeYtoX", "transposeYtoZ", "transposeZtoY",
           "transposeXtoZ", "transposeZtoX"]
