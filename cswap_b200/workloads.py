"""The two training-step workloads the swap path is measured on, wrapped layer
by layer in Execution.pre/post exactly the way the reference's drivers do.

* VGG16 for 3x32x32 inputs: the 45-layer list, the flatten / fc / loss tail and
  the tensor-id convention (id = index of the producing layer, swapped when the
  next layer consumes it) of CSWAP+/vgg16-cifar10.cpp:77-245,381-397.
* A BERT-style encoder with every linear / matmul / softmax / dropout /
  layer-norm / activation wrapped, as CSWAP+/bert.cpp:370-801 does, with the
  dimensions left to the caller (the benchmark uses the BERT-base shape).

Inputs are synthetic (the datasets are not part of this repository) and
weights are randomly initialised.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .codec import POLICY_KEEP, POLICY_RAW, POLICY_ZFP
from .execution import Execution, LayerType


# ---------------------------------------------------------------------------
# VGG16 (vgg16-cifar10.cpp:77-178)
# ---------------------------------------------------------------------------
_VGG_CFG = [64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M"]

# the conv inputs the reference compresses (vgg16-cifar10.cpp:396-397)
VGG_CONV_INPUT_IDS = (2, 6, 9, 13, 16, 19, 23, 26, 29, 33, 36, 39)


class VGG16(nn.Module):
    def __init__(self, num_classes: int = 10):
        super().__init__()
        layers: List[nn.Module] = []
        types: List[LayerType] = []
        c_in = 3
        for v in _VGG_CFG:
            if v == "M":
                layers.append(nn.MaxPool2d(2))
                types.append(LayerType.POOL)
            else:
                layers += [nn.Conv2d(c_in, v, 3, padding=1), nn.BatchNorm2d(v), nn.ReLU()]
                types += [LayerType.CONV, LayerType.BN, LayerType.ACT]
                c_in = v
        layers.append(nn.AvgPool2d(1))
        types.append(LayerType.POOL)
        assert len(layers) == 45
        self.features = nn.ModuleList(layers)
        self.types = types
        self.fc1 = nn.Linear(512, num_classes)

    def forward_with(self, exe: Execution, x: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        """vgg16-cifar10.cpp:215-245."""
        pre = x
        exe.preforward()
        for layer, lt in zip(self.features, self.types):
            exe.pre(pre, lt)
            out = layer(pre)
            exe.post(pre, out, lt, False, _stateless(layer))
            pre = out
        exe.pre(pre)
        out = pre.view(pre.size(0), -1)
        exe.post(pre, out, LayerType.ACT, True)
        pre = out
        exe.pre(pre)
        out = self.fc1(pre)
        exe.post(pre, out, LayerType.FC, True)
        pre = out
        exe.pre([pre, target])
        loss = F.cross_entropy(pre, target)
        exe.post([pre, target], loss, LayerType.ACT, True)
        exe.postforward()
        return loss


def _stateless(layer: nn.Module):
    """The layer as a function that can be run a second time in backward to
    rebuild a dropped output: BatchNorm without its running statistics (the
    training-mode output does not depend on them), everything else as is."""
    if isinstance(layer, nn.BatchNorm2d):
        return lambda t, m=layer: F.batch_norm(t, None, None, m.weight, m.bias, True, 0.0, m.eps)
    return layer


def vgg16_baseline_policy(exe: Execution, planner: int) -> None:
    """The baseline planners as the reference's drivers set them up
    (Desnet-cifar10.cpp:732-745): an all-zero policy table with `policy_` 3 (vDNN:
    raw swap of every conv input) or 4 (SuperNeurons: the same, and the inputs
    of all other layers dropped and rebuilt)."""
    n = len(exe.policy)
    for i in range(min(50, n)):
        exe.begin_stage[i] = i + 1
        exe.policy[i] = POLICY_KEEP
    exe.policy_ = planner


def vgg16_reference_policy(exe: Execution, compressed: int = POLICY_ZFP) -> None:
    """The hard-wired setting of vgg16-cifar10.cpp:381-397: every tensor is
    swapped when the next layer consumes it, the twelve conv inputs with
    `compressed`, the rest raw."""
    n = len(exe.policy)
    for i in range(min(50, n)):
        exe.begin_stage[i] = i + 1
        exe.policy[i] = POLICY_RAW
    for i in VGG_CONV_INPUT_IDS:
        exe.policy[i] = compressed


# ---------------------------------------------------------------------------
# BERT-style encoder (bert.cpp:370-801)
# ---------------------------------------------------------------------------
class BertEncoder(nn.Module):
    def __init__(self, vocab: int = 30522, hidden: int = 768, layers: int = 12, heads: int = 12, ffn: int = 3072,
                 max_seq: int = 512, dropout: float = 0.1):
        super().__init__()
        self.hidden, self.heads, self.nlayers, self.p = hidden, heads, layers, dropout
        self.tok = nn.Embedding(vocab, hidden)
        self.pos = nn.Embedding(max_seq, hidden)
        self.emb_ln = nn.LayerNorm(hidden)
        self.q = nn.ModuleList(nn.Linear(hidden, hidden) for _ in range(layers))
        self.k = nn.ModuleList(nn.Linear(hidden, hidden) for _ in range(layers))
        self.v = nn.ModuleList(nn.Linear(hidden, hidden) for _ in range(layers))
        self.o = nn.ModuleList(nn.Linear(hidden, hidden) for _ in range(layers))
        self.ln1 = nn.ModuleList(nn.LayerNorm(hidden) for _ in range(layers))
        self.f1 = nn.ModuleList(nn.Linear(hidden, ffn) for _ in range(layers))
        self.f2 = nn.ModuleList(nn.Linear(ffn, hidden) for _ in range(layers))
        self.ln2 = nn.ModuleList(nn.LayerNorm(hidden) for _ in range(layers))
        self.head = nn.Linear(hidden, 2)

    def forward_with(self, exe: Execution, ids: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        B, S = ids.shape
        H, nh = self.hidden, self.heads
        dh = H // nh

        def step(fn: Callable, inputs, lt=LayerType.ACT, omit=False):
            exe.pre(inputs, lt)
            out = fn(*inputs) if isinstance(inputs, (list, tuple)) else fn(inputs)
            exe.post(inputs, out, lt, omit)
            return out

        exe.preforward()
        pos = torch.arange(S, device=ids.device).unsqueeze(0).expand(B, S)
        x = step(lambda i: self.tok(i) + self.pos(pos), ids, LayerType.ACT, True)
        x = step(self.emb_ln, x, LayerType.BN)
        x = step(lambda t: F.dropout(t, self.p, self.training), x)
        for l in range(self.nlayers):
            q = step(self.q[l], x, LayerType.FC)
            k = step(self.k[l], x, LayerType.FC)
            v = step(self.v[l], x, LayerType.FC)
            qh = step(lambda t: t.view(B, S, nh, dh).transpose(1, 2).contiguous(), q)
            kh = step(lambda t: t.view(B, S, nh, dh).permute(0, 2, 3, 1).contiguous(), k)
            vh = step(lambda t: t.view(B, S, nh, dh).transpose(1, 2).contiguous(), v)
            sc = step(lambda a, b: torch.matmul(a, b) * (dh ** -0.5), [qh, kh], LayerType.FC)
            pr = step(lambda t: torch.softmax(t, dim=-1), sc)
            pr = step(lambda t: F.dropout(t, self.p, self.training), pr)
            ctx = step(lambda a, b: torch.matmul(a, b), [pr, vh], LayerType.FC)
            ctx = step(lambda t: t.transpose(1, 2).reshape(B, S, H), ctx)
            ao = step(self.o[l], ctx, LayerType.FC)
            ao = step(lambda t: F.dropout(t, self.p, self.training), ao)
            x = step(lambda a, b: self.ln1[l](a + b), [ao, x], LayerType.BN)
            h = step(self.f1[l], x, LayerType.FC)
            h = step(F.gelu, h)
            h = step(self.f2[l], h, LayerType.FC)
            h = step(lambda t: F.dropout(t, self.p, self.training), h)
            x = step(lambda a, b: self.ln2[l](a + b), [h, x], LayerType.BN)
        cls = step(lambda t: t[:, 0], x, LayerType.ACT, True)
        logits = step(self.head, cls, LayerType.FC, True)
        loss = step(lambda a, b: F.cross_entropy(a, b), [logits, target], LayerType.ACT, True)
        exe.postforward()
        return loss


# ---------------------------------------------------------------------------
# measuring a swapped step
# ---------------------------------------------------------------------------
def timed_steps(model: nn.Module, exe: Execution, make_batch: Callable[[], Tuple[torch.Tensor, torch.Tensor]],
                steps: int, warmup: int) -> dict:
    """Run forward + backward `steps` times under `exe`'s policy.  Each step
    takes its batch from pinned host memory (non-blocking copy) and reads the
    loss back, so the numbers include the step's host traffic."""
    times = []
    loss_val = float("nan")
    exe.mgr.reset_stats()
    for it in range(warmup + steps):
        if it == warmup:
            torch.cuda.synchronize()
            exe.mgr.reset_stats()
            torch.cuda.reset_peak_memory_stats()
        hx, hy = make_batch()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        x = hx.cuda(non_blocking=True)
        y = hy.cuda(non_blocking=True)
        if x.is_floating_point():
            x.requires_grad_(True)  # the first layer's input has a grad_fn-less leaf; keep autograd on throughout
        for p in model.parameters():
            p.grad = None
        loss = model.forward_with(exe, x, y)
        loss.backward()
        loss_val = float(loss.detach())  # device -> host read of the step's result
        e1.record()
        torch.cuda.synchronize()
        if it >= warmup:
            times.append(e0.elapsed_time(e1))
    exe.mgr.sync()
    s = exe.mgr.stats()
    n = max(steps, 1)
    times.sort()
    return {"ms_per_step": sum(times) / n, "ms_median": times[len(times) // 2], "loss": loss_val,
            "swapped_tensors_per_step": s["swap_outs"] / n, "activation_bytes_per_step": s["raw_bytes_out"] / n,
            "activation_bytes_back_per_step": s["raw_bytes_in"] / n,
            "link_bytes_out_per_step": s["moved_bytes_out"] / n, "link_bytes_in_per_step": s["moved_bytes_in"] / n,
            "pinned_high_water": s["pinned_high_water"], "staging_high_water": s["staging_high_water"],
            "peak_device_bytes": torch.cuda.max_memory_allocated(),
            "dropped_tensors_per_step": exe.dropped_tensors / max(warmup + steps, 1),
            "recomputed_tensors_per_step": exe.recomputed_tensors / max(warmup + steps, 1)}
