"""cswap_b200: B200-native compressed tensor-swap path (ZFP fixed-rate and
zero-value sparse codecs, swap manager, cost model) behind a C ABI.

The CUDA library is the only implementation: importing the codec functions
without ``libcswap_b200.so`` raises, there is no CPU path.
"""
from ._lib import lib, LibraryMissing, CswapError, check  # noqa: F401
from .codec import (  # noqa: F401
    POLICY_KEEP, POLICY_DROP, POLICY_RAW, POLICY_SPARSE, POLICY_ZFP,
    zfp_max_bytes, zfp_compress, zfp_decompress, zfp_view,
    sparse_layout, sparse_compress, sparse_decompress, sparse_packed_bytes,
    legacy_sparse_compress, legacy_sparse_decompress,
)
from .swap import SwapManager, Ticket, CostModel, TensorDesc, blob_info  # noqa: F401
from .execution import Execution, LayerType  # noqa: F401

__version__ = "0.1.0"
