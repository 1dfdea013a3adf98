"""The hook functions the reference's modified PyTorch exposes to its Python
model zoo, on stock PyTorch.

The reference's drivers call `torch.cswapinit_()` once, `torch.cswapinit()` at
the top of every forward pass, `torch.cswapsetratio(r)`, and wrap each layer as

    torch.cswappre(pre, type); out = layer(pre); torch.cswappost(pre, out, type)

(CIFAR10/cifar10.py:86,106, CIFAR10/models/vgg.py:23-46), where `type` is the
policy for the layer's input: 0 keep, 2 raw swap, 3 sparse, 6 ZFP.  Here the
same five names are module functions over one process-wide `Execution`:

    import cswap_b200.compat as cswap
    cswap.cswapinit_()
    ...
    cswap.cswappre(pre, 6); out = conv(pre); cswap.cswappost(pre, out, 6)

`install(torch)` additionally sets them as attributes of the torch module, so
that a model file written for the reference runs unchanged.
"""
from __future__ import annotations

from typing import Optional

import torch

from .codec import POLICY_DROP, POLICY_KEEP, POLICY_RAW, POLICY_SPARSE, POLICY_ZFP
from .execution import Execution, LayerType
from .swap import SwapManager

_exe: Optional[Execution] = None
_MAX_IDS = 1 << 16


def execution() -> Execution:
    """The process-wide Execution behind the hook functions."""
    if _exe is None:
        raise RuntimeError("call cswapinit_() first")
    return _exe


def cswapinit_(mgr: Optional[SwapManager] = None, zfp_maxbits: Optional[int] = None) -> None:
    """Once per process (cifar10.py:86): pools, streams, tables."""
    global _exe
    if _exe is not None and _exe.mgr is not None and _exe.mgr is not mgr:
        _exe.postforward()
    _exe = Execution(mgr=mgr)
    _exe.init_(_MAX_IDS, zfp_maxbits)


def cswapsetratio(maxbits: int) -> None:
    """Bits per zfp block for the tensors swapped from now on (cifar10.py:106)."""
    execution().set_ratio(int(maxbits))


def cswapinit() -> None:
    """Top of every forward pass (models/vgg.py:23)."""
    execution().preforward()


def cswappre(pre: torch.Tensor, type: int = 0) -> None:  # noqa: A002 - the reference's parameter name
    """Before the layer that consumes `pre`: start swapping it out under policy
    `type` (models/vgg.py:38-41).  A tensor no wrapped layer produced (the
    network input) has no id and stays."""
    exe = execution()
    tid = getattr(pre, "tensor_id", -1)
    if 0 <= tid < _MAX_IDS:
        exe.policy[tid] = int(type) if int(type) in (POLICY_DROP, POLICY_RAW, POLICY_SPARSE, POLICY_ZFP) \
            else POLICY_KEEP
        exe.begin_stage[tid] = exe.index + 1
    exe.pre(pre, LayerType.ACT)


def cswappost(pre: torch.Tensor, out: torch.Tensor, type: int = 0, forward=None) -> None:  # noqa: A002
    """After the layer: `out` gets its id, `pre`'s device copy is let go
    (models/vgg.py:42-43)."""
    exe = execution()
    if exe.index >= _MAX_IDS:
        raise RuntimeError("more wrapped layers in one forward pass than ids")
    exe.post(pre, out, LayerType.ACT, False, forward)


def install(module=torch) -> None:
    """Make the five functions attributes of `module` (default: torch itself)."""
    for fn in (cswapinit_, cswapinit, cswapsetratio, cswappre, cswappost):
        setattr(module, fn.__name__, fn)
