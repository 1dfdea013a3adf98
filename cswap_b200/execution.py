"""Host-side mirror of the reference's swap orchestrator.

`Execution` keeps the interface the CSWAP+ model drivers use
(CSWAP+/Execution.h:38-447): `init_`, `preforward`, `pre`, `post`,
`postforward`, the public tables `policy`, `begin_stage`, `index`, `policy_`,
and the policy codes 0 keep / 1 drop and recompute / 2 raw / 3 sparse / 6 ZFP.
A driver wraps every layer as

    exe.pre(x)            # may start swapping x out (Execution.h:65-133)
    y = layer(x)
    exe.post(x, y)        # y.tensor_id = index; x's device copy is let go
                          # (Execution.h:217-310)

and brackets the forward pass with `preforward()` / `postforward()`.

Policy 1 (Execution.h:243-247 clears the storage and leaves the rebuilding to
the modified engine, which is not part of the reference tree): `post` takes
the layer as an extra argument, `post(x, y, type, isomit, forward=layer)`, and a
dropped tensor is rebuilt in backward by running its producer again on the
producer's own input, which is in turn swapped in or rebuilt as needed.  Only
stateless callables may be passed (a BatchNorm module would update its running
statistics a second time; pass a closure over F.batch_norm without them).  A
tensor whose producer was not given stays on the device.  `policy_` 3 and 4
select the vDNN and SuperNeurons baselines as in Execution.h:70,243,248.

The reference swaps the storage's DataPtr under the autograd graph and relies
on a modified engine to bring it back.  On stock PyTorch the same effect is
reached with saved-tensor hooks that stay installed for the whole forward
pass: every activation autograd saves is held through a small record keyed by
its storage; when `pre` swaps a tensor out, the record lets go of the device
copy (the memory returns to the allocator once the driver's own reference is
gone) and the first use in backward swaps it back in, prefetching the
previously swapped tensor's payload one step ahead.
"""
from __future__ import annotations

import enum
import weakref
from typing import Dict, List, Optional, Sequence, Union

import torch

from .codec import POLICY_DROP, POLICY_KEEP, POLICY_RAW, POLICY_SPARSE, POLICY_ZFP
from ._lib import CswapError
from .swap import CostModel, SwapManager, TensorDesc, Ticket


class LayerType(enum.IntEnum):
    """CSWAP+/Execution.h:28-35."""
    CONV = 0
    POOL = 1
    ACT = 2
    BN = 3
    FC = 4
    MASKFILL = 5


class _Record:
    """Residency of one activation storage: on the device (`tensor`) or
    swapped out (`ticket`)."""

    __slots__ = ("tensor", "ticket", "numel", "order", "exe", "producer", "dropped", "saved", "ahead",
                 "__weakref__")

    def __init__(self, tensor: torch.Tensor, exe: "Execution"):
        self.tensor: Optional[torch.Tensor] = tensor
        self.ticket: Optional[Ticket] = None
        self.numel = tensor.numel()
        self.order = -1
        self.exe = weakref.ref(exe)
        self.producer = None   # (callable, packed inputs) when the driver passed the layer to post()
        self.dropped = False   # policy 1: let go without a copy, rebuilt by `producer`
        self.saved = False     # autograd holds it for backward (a pack hook has seen it)
        self.ahead = None      # destination of a swap-in started before the tensor was asked for

    def materialize(self) -> torch.Tensor:
        if self.tensor is None:
            exe = self.exe()
            if self.ticket is not None and self.ahead is not None:
                exe.mgr.swap_in_wait(self.ticket)   # copy and decode were started one step earlier
                self.tensor, self.ahead = self.ahead.view(-1), None
                exe._after_swap_in(self)
            elif self.ticket is not None:
                back = exe.mgr.reclaim(self.ticket)
                if back is not None:
                    # needed again before it had left the device: take it back as it is
                    self.tensor = back.view(-1)
                    self.ticket = None
                else:
                    self.tensor = exe.mgr.swap_in(self.ticket).view(-1)
                exe._after_swap_in(self)
            else:
                fn, packed = self.producer
                with torch.no_grad():
                    out = fn(*[exe._unpack(p) for p in packed])
                if out.numel() != self.numel or out.dtype != torch.float32:
                    raise RuntimeError("recomputed activation does not match the dropped one")
                self.tensor = out.detach().contiguous().view(-1)
                exe.recomputed_tensors += 1
        return self.tensor

    def __del__(self):
        t = self.ticket
        if self.ahead is not None and t is not None:
            # a swap-in started ahead of time that nobody waited for may still be writing its tensor
            try:
                self.exe().mgr.sync()
            except Exception:
                pass
        if t is not None:
            try:
                t.release()
            except Exception:
                pass


class _Packed:
    __slots__ = ("rec", "shape", "stride", "offset")

    def __init__(self, rec, shape, stride, offset):
        self.rec, self.shape, self.stride, self.offset = rec, shape, stride, offset


TensorOrList = Union[torch.Tensor, Sequence[torch.Tensor]]


class Execution:
    def __init__(self, mgr: Optional[SwapManager] = None, min_numel: int = 1024):
        self.mgr = mgr
        self.index = -1
        self.policy: List[int] = []
        self.begin_stage: List[int] = []
        self.types: List[LayerType] = []
        self.policy_ = 1  # 1 CSWAP, 2 Capuchin, 3 vDNN, 4 SuperNeurons (Execution.h:420)
        self.min_numel = min_numel
        self.profile = False
        self._records: "weakref.WeakValueDictionary[int, _Record]" = weakref.WeakValueDictionary()
        self._pending: List[_Record] = []
        self._swapped: List["weakref.ref[_Record]"] = []
        self._produced: List[_Record] = []  # keeps producer notes alive until autograd holds the records
        self._deferred: List[tuple] = []    # (record, policy): swap only if the running layer saves the tensor
        self.skipped_unsaved = 0
        self._hooks = None
        self._prof: Dict[int, dict] = {}
        self._prof_saved: Dict[int, bool] = {}
        self._prof_start = None
        self.swapped_tensors = 0
        self.dropped_tensors = 0
        self.recomputed_tensors = 0
        self.skipped_for_memory = 0

    # ---- set-up (Execution.h:46-64) -------------------------------------------
    def init_(self, n: int, zfp_maxbits: Optional[int] = None) -> None:
        self.policy = [POLICY_KEEP] * n
        self.begin_stage = [0] * n
        if self.mgr is None:
            self.mgr = SwapManager()
        if zfp_maxbits is not None:
            self.mgr.set_zfp_maxbits(zfp_maxbits)

    def set_ratio(self, maxbits: int) -> None:
        """The reference's setRatio(bits per zfp block), Execution.h:63."""
        self.mgr.set_zfp_maxbits(maxbits)

    # ---- per step (Execution.h:403-412) ----------------------------------------
    def preforward(self) -> None:
        self.index = -1
        self._pending.clear()
        self._swapped.clear()
        self._produced.clear()
        self._deferred.clear()
        if self._hooks is None:
            self._hooks = torch.autograd.graph.saved_tensors_hooks(self._pack, self._unpack)
            self._hooks.__enter__()

    def postforward(self) -> None:
        if self._hooks is not None:
            self._hooks.__exit__(None, None, None)
            self._hooks = None
        self._pending.clear()
        self._produced.clear()

    # ---- saved-tensor hooks ------------------------------------------------------
    def _key(self, t: torch.Tensor) -> Optional[int]:
        """Address of t's storage when t is a whole, contiguous float32 CUDA
        storage worth tracking, else None (one storage lookup for both answers)."""
        if not (t.is_cuda and t.dtype == torch.float32 and t.numel() >= self.min_numel and t.is_contiguous()
                and t.storage_offset() == 0) or (t.is_leaf and t.requires_grad):
            return None
        st = t.untyped_storage()
        return st.data_ptr() if st.nbytes() == t.numel() * 4 else None

    def _eligible(self, t: torch.Tensor) -> bool:
        return self._key(t) is not None

    def _record_for(self, t: torch.Tensor, key: Optional[int] = None) -> _Record:
        if key is None:
            key = t.untyped_storage().data_ptr()
        rec = self._records.get(key)
        if rec is None or rec.tensor is None or rec.numel != t.numel() \
                or rec.tensor.untyped_storage().data_ptr() != key:
            rec = _Record(t.detach().view(-1), self)
            self._records[key] = rec
        return rec

    def _pack(self, t: torch.Tensor):
        key = self._key(t)
        if key is None:
            return t
        rec = self._record_for(t, key)
        rec.saved = True
        return _Packed(rec, t.shape, t.stride(), 0)

    def _ref(self, t: torch.Tensor):
        """Like _pack, for the producer notes: a way back to the tensor that does
        not count as autograd having saved it."""
        key = self._key(t)
        if key is None:
            return t
        return _Packed(self._record_for(t, key), t.shape, t.stride(), 0)

    def _unpack(self, p):
        if not isinstance(p, _Packed):
            return p
        return p.rec.materialize().as_strided(p.shape, p.stride, p.offset)

    def _after_swap_in(self, rec: _Record) -> None:
        # one step ahead: start bringing back the tensor swapped out just before
        for i in range(rec.order - 1, -1, -1):
            r = self._swapped[i]() if i < len(self._swapped) else None
            if r is not None and r.tensor is None and r.ticket is not None:
                # a lossless ticket still on its way out may yet be taken back whole
                if (r.ticket.policy == POLICY_ZFP or self.mgr.out_done(r.ticket)) and r.ahead is None:
                    # copy AND decode, into a tensor taken now, so that the consumer's backward
                    # finds it ready instead of waiting for a decode that starts when it asks
                    r.ahead = self.mgr.swap_in_start(r.ticket)
                break

    # ---- pre / post ----------------------------------------------------------------
    def _effective_policy(self, tid: int, layer_type: LayerType) -> int:
        pol = self.policy[tid] if tid < len(self.policy) else POLICY_KEEP
        if pol == POLICY_DROP or (self.policy_ == 4 and layer_type != LayerType.CONV):
            return POLICY_DROP  # Execution.h:243: SuperNeurons rebuilds the inputs of non-conv layers
        if layer_type == LayerType.CONV and self.policy_ > 2:
            return POLICY_RAW  # vDNN / SuperNeurons baselines (Execution.h:70,248)
        return pol

    def pre(self, x: TensorOrList, layer_type: LayerType = LayerType.ACT) -> None:
        self.index += 1
        inputs = [x] if isinstance(x, torch.Tensor) else list(x)
        for t in inputs:
            tid = getattr(t, "tensor_id", -1)
            if tid < 0 or tid >= len(self.begin_stage) or self.index != self.begin_stage[tid] or t.grad_fn is None:
                continue
            pol = self._effective_policy(tid, layer_type)
            if pol not in (POLICY_DROP, POLICY_RAW, POLICY_SPARSE, POLICY_ZFP):
                continue
            key = self._key(t)
            if key is None:
                continue
            rec = self._record_for(t, key)
            if rec.ticket is not None or rec.dropped:
                continue
            if pol == POLICY_DROP:
                if rec.producer is not None:  # without its producer the tensor simply stays
                    rec.dropped = True
                    self._pending.append(rec)
                    self.dropped_tensors += 1
                continue
            if not rec.saved:
                # Nothing has saved this tensor for backward yet.  Only the layer about to
                # run still can (this is its last forward use): copy it out afterwards if it
                # did, and not at all if it did not - it is dead then and dies by itself.
                self._deferred.append((rec, pol))
                continue
            self._start_swap(rec, pol)
        if self.profile:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._prof_start = ev

    def _start_swap(self, rec: _Record, pol: int) -> None:
        try:
            rec.ticket = self.mgr.swap_out(rec.tensor, pol)
        except CswapError as err:
            if err.status != 4:  # pools exhausted: this tensor simply stays on the device
                raise
            self.skipped_for_memory += 1
            return
        rec.order = len(self._swapped)
        self._swapped.append(weakref.ref(rec))
        self._pending.append(rec)
        self.swapped_tensors += 1

    def post(self, x: TensorOrList, y: torch.Tensor, layer_type: LayerType = LayerType.ACT,
             isomit: bool = False, forward=None) -> None:
        y.tensor_id = self.index
        inputs = [x] if isinstance(x, torch.Tensor) else list(x)
        if forward is not None and self._hooks is not None and self._eligible(y) and not any(
                t.is_cuda and t.untyped_storage().data_ptr() == y.untyped_storage().data_ptr() for t in inputs):
            # how to rebuild y should it be dropped: its producer and the producer's inputs
            # (a view of an input shares the input's record and is rebuilt with it)
            rec = self._record_for(y)
            rec.producer = (forward, [self._ref(t) for t in inputs])
            self._produced.append(rec)
        if self.profile:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            zf = (y.detach() == 0).float().mean() if (y.is_cuda and y.dtype == torch.float32) else None
            self._prof[self.index] = {
                "start": self._prof_start, "end": ev, "numel": y.numel(), "zero_fraction": zf,
                "inputs": [getattr(t, "tensor_id", -1) for t in inputs], "omit": isomit,
                "type": int(layer_type), "float32": y.dtype == torch.float32, "has_grad": y.grad_fn is not None,
                "recomputable": forward is not None, "bwd": None,
            }
            if y.grad_fn is not None:
                # when this layer's backward begins: what a tensor it consumed has to be back by
                def mark(_grads, idx=self.index):
                    rec = self._prof.get(idx)
                    if rec is not None and rec["bwd"] is None:
                        e = torch.cuda.Event(enable_timing=True)
                        e.record()
                        rec["bwd"] = e
                y.grad_fn.register_prehook(mark)
            # which consumed tensors autograd holds on to once this consumer has run
            for t in inputs:
                tid = getattr(t, "tensor_id", -1)
                if tid >= 0 and isinstance(t, torch.Tensor) and self._eligible(t):
                    rec = self._records.get(t.untyped_storage().data_ptr())
                    self._prof_saved[tid] = bool(rec is not None and rec.saved)
        for rec, pol in self._deferred:
            if rec.saved and rec.ticket is None and rec.tensor is not None:
                self._start_swap(rec, pol)
            elif not rec.saved:
                self.skipped_unsaved += 1
        self._deferred.clear()
        # the layer has run and saved what it needs: let go of the device copies
        for rec in self._pending:
            rec.tensor = None
        self._pending.clear()

    # ---- self-tuning policy (call sites Execution.h:224-233, resnet-cifar10.cpp:407-437) ---
    def finish_profile(self) -> Dict[int, dict]:
        """Turn the events of a profiled iteration into numbers (synchronises)."""
        torch.cuda.synchronize()
        out = {}
        marks = [i for i in sorted(self._prof) if self._prof[i].get("bwd") is not None]
        first = self._prof[marks[-1]]["bwd"] if marks else None  # backward starts at the last layer
        for idx, p in self._prof.items():
            out[idx] = {
                "bwd_start_s": first.elapsed_time(p["bwd"]) * 1e-3 if first is not None and p.get("bwd") is not None
                else -1.0,
                "time_s": p["start"].elapsed_time(p["end"]) * 1e-3, "numel": p["numel"],
                "zero_fraction": float(p["zero_fraction"]) if p["zero_fraction"] is not None else -1.0,
                "inputs": p["inputs"], "omit": p["omit"], "type": p["type"], "float32": p["float32"],
                "has_grad": p["has_grad"], "saved": self._prof_saved.get(idx, True),
                "recomputable": p.get("recomputable", False),
            }
        self._prof = {}
        self._prof_saved = {}
        self.profile = False
        return out

    def _candidates(self, prof: Dict[int, dict], lossy_ids, bwd_factor: float, min_bytes: int):
        """Swap candidates of a profiled iteration with what the cost model needs to know about each."""
        n = max(prof) + 1 if prof else 0
        times = [prof[i]["time_s"] if i in prof else 0.0 for i in range(n)]
        start = [0.0] * (n + 1)
        for i in range(n):
            start[i + 1] = start[i] + times[i]
        fwd_total = start[n]
        consumer: Dict[int, int] = {}
        conv_inputs = set()
        for idx in sorted(prof):
            for tid in prof[idx]["inputs"]:
                if tid >= 0 and tid not in consumer:
                    consumer[tid] = idx
                    if prof[idx]["type"] == int(LayerType.CONV):
                        conv_inputs.add(tid)
        lossy = set(lossy_ids) if lossy_ids is not None else conv_inputs
        if len(self.policy) < n:
            self.policy += [POLICY_KEEP] * (n - len(self.policy))
            self.begin_stage += [0] * (n - len(self.begin_stage))
        cands, descs = [], []
        for tid in sorted(consumer, key=lambda t: consumer[t]):
            p = prof.get(tid)
            if p is None or p["omit"] or not p["float32"] or not p["has_grad"] or p["numel"] * 4 < min_bytes:
                continue
            if not p.get("saved", True):
                continue  # nothing keeps it for backward: it dies after its consumer and costs no link time
            c = consumer[tid]
            cands.append(tid)
            # needed when the consumer's backward begins: measured where the profiled iteration
            # ran backward, else estimated from the forward times of the later layers
            measured = prof.get(c, {}).get("bwd_start_s", -1.0)
            need = measured if measured >= 0 else bwd_factor * (fwd_total - start[c + 1])
            descs.append(TensorDesc(p["numel"], p["zero_fraction"], tid in lossy, ready_s=start[c], need_s=need))
        return n, fwd_total, consumer, cands, descs

    def make_policy(self, prof: Dict[int, dict], cost: CostModel, lossy_ids: Optional[Sequence[int]] = None,
                    bwd_factor: float = 2.0, min_bytes: int = 1 << 20) -> List[int]:
        """Fill `policy` / `begin_stage` from a profiled iteration.

        Tensor id i (the output of layer i) becomes a swap candidate at the
        first layer that consumes it.  The cost model gets, per candidate, the
        forward time at which that consumer starts and the backward compute
        that precedes the consumer's backward (taken as `bwd_factor` times the
        forward time of the layers after it), and simulates the step's link
        traffic to choose raw / sparse / ZFP.  ZFP is allowed on the ids in
        `lossy_ids` (default: inputs of CONV layers, which is where the
        reference's drivers apply it, vgg16-cifar10.cpp:381-397)."""
        n, fwd_total, consumer, cands, descs = self._candidates(prof, lossy_ids, bwd_factor, min_bytes)
        pol, _ = cost.decide(descs, fwd_total)
        for tid in range(n):
            self.policy[tid] = POLICY_KEEP
        for tid, pcode in zip(cands, pol):
            self.policy[tid] = pcode
            self.begin_stage[tid] = consumer[tid]
        return list(self.policy)

    def make_policy_capuchin(self, prof: Dict[int, dict], cost: CostModel, bwd_factor: float = 2.0,
                             min_bytes: int = 1 << 20) -> List[int]:
        """A swap-or-recompute table in the manner of the Capuchin baseline
        (`policy_` 2; the reference takes its table from the fork's
        PolicyMaker::capuchin, vgg16-style drivers at Desnet-cifar10.cpp:723-731,
        which is not part of the tree).  Every candidate starts as a raw swap;
        the step is simulated on the measured link, and while some tensor's
        modelled stall exceeds the forward time of the layer that produced it,
        the worst such tensor is dropped and rebuilt instead (policy 1) and the
        simulation repeated.  Only tensors whose producer was passed to `post`
        during the profiled iteration can be rebuilt."""
        n, fwd_total, consumer, cands, descs = self._candidates(prof, [], bwd_factor, min_bytes)
        for d in descs:
            d.zero_fraction = -1.0  # no codec: Capuchin moves tensors as they are
        active = list(range(len(cands)))
        dropped = set()
        while active:
            _, stall = cost.decide([descs[i] for i in active], fwd_total)
            best, gain = -1, 0.0
            for j, i in enumerate(active):
                p = prof[cands[i]]
                if p.get("recomputable") and stall[j] - p["time_s"] > gain:
                    best, gain = i, stall[j] - p["time_s"]
            if best < 0:
                break
            dropped.add(best)
            active.remove(best)
        for tid in range(n):
            self.policy[tid] = POLICY_KEEP
        for i, tid in enumerate(cands):
            self.policy[tid] = POLICY_DROP if i in dropped else POLICY_RAW
            self.begin_stage[tid] = consumer[tid]
        self.policy_ = 2
        return list(self.policy)

    def policy_candidates(self, prof: Dict[int, dict], cost: CostModel, lossy_ids: Optional[Sequence[int]] = None,
                          bwd_factor: float = 2.0, min_bytes: int = 1 << 20) -> Dict[str, List[int]]:
        """The cost model's table and its neighbour with ZFP on every tensor
        where loss is allowed.  The model minimises the stall it can predict
        from the profile; on a step that is bound by the host link or by the
        host itself it predicts too little, and the neighbour is then the
        faster one.  `refine_policy` settles it by measurement."""
        model = self.make_policy(prof, cost, lossy_ids, bwd_factor, min_bytes)
        begin = list(self.begin_stage)
        _, _, consumer, cands, descs = self._candidates(prof, lossy_ids, bwd_factor, min_bytes)
        eager = list(model)
        for tid, d in zip(cands, descs):
            if d.lossy_ok and d.numel >= 1024:
                eager[tid] = POLICY_ZFP
        self.begin_stage = begin
        return {"model": model, "zfp_where_allowed": eager}

    def refine_policy(self, candidates: Dict[str, List[int]], run_steps, steps: int = 3) -> str:
        """Install the candidate table that runs fastest: `run_steps(n)` must
        run n training steps under this Execution and return the seconds they
        took.  Returns the winner's name.  (One untimed step per candidate
        first: the pools and the allocator settle on the new traffic.)"""
        best_name, best_t = None, float("inf")
        for name, table in candidates.items():
            self.policy[:len(table)] = table
            run_steps(1)
            t = run_steps(steps)
            if t < best_t:
                best_name, best_t = name, t
        self.policy[:len(candidates[best_name])] = candidates[best_name]
        return best_name

