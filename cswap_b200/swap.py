"""Python face of the swap manager and cost model (section 4 and 5 of
include/cswap_b200.h)."""
from __future__ import annotations

import ctypes as C
import json
from dataclasses import dataclass
from typing import Iterable, List, Optional, Sequence, Tuple

import torch

from ._lib import (BlobHeader, CostModelStruct, MgrConfig, MgrStats, TensorDescStruct, TicketInfo, check, lib)
from .codec import POLICY_RAW, POLICY_SPARSE, POLICY_ZFP, _require_cuda_f32, _stream_ptr


def blob_info(blob) -> dict:
    """Header of a self-describing blob after validation (needs no GPU)."""
    import numpy as np
    a = np.ascontiguousarray(np.frombuffer(blob, dtype=np.uint8) if not isinstance(blob, np.ndarray) else blob)
    h = BlobHeader()
    check(lib().csw_blob_info(a.ctypes.data, a.size, C.byref(h)), "csw_blob_info")
    return {"policy": h.policy, "numel": h.numel, "zfp_maxbits": h.zfp_maxbits, "payload_bytes": h.payload_bytes,
            "nnz": h.nnz, "version": h.version}


class _Parked:
    """Handle of a given-up ticket whose source tensor the device still reads."""
    __slots__ = ("_h", "policy")

    def __init__(self, h, policy):
        self._h, self.policy = h, policy


class Ticket:
    """One swapped-out tensor.  Holds the handle and what is needed to
    rebuild the tensor (shape, device)."""

    __slots__ = ("_mgr", "_h", "shape", "numel", "device", "policy", "__weakref__")

    def __init__(self, mgr: "SwapManager", handle: int, shape, numel: int, device, policy: int = -1):
        self._mgr, self._h, self.shape, self.numel, self.device = mgr, handle, tuple(shape), numel, device
        self.policy = policy  # as requested by the caller

    @property
    def alive(self) -> bool:
        return self._h is not None

    def info(self) -> dict:
        ti = TicketInfo()
        check(lib().csw_ticket_query(self._mgr._h, self._h, C.byref(ti)), "csw_ticket_query")
        return {"policy": ti.policy, "numel": ti.numel, "raw_bytes": ti.raw_bytes, "moved_bytes": ti.moved_bytes,
                "complete": bool(ti.complete)}

    def export(self):
        """The swapped-out tensor as a self-describing blob (numpy uint8 array):
        a 64-byte header (policy, element count, zfp bits per block, sparse
        count) and the payload as it crossed the link.  Waits for the copy out."""
        import numpy as np
        n = C.c_size_t()
        check(lib().csw_ticket_export(self._mgr._h, self._h, None, 0, C.byref(n)), "csw_ticket_export")
        buf = np.empty(n.value, dtype=np.uint8)
        check(lib().csw_ticket_export(self._mgr._h, self._h, buf.ctypes.data, buf.size, C.byref(n)),
              "csw_ticket_export")
        return buf

    def release(self) -> None:
        """Give the ticket up; its pool memory returns once its copies have
        finished.  Never blocks: if the device is still reading the source
        tensor, ticket and tensor are parked and retired by a later call."""
        mgr = self._mgr
        if self._h is not None and mgr._h is not None:
            for i, (tk, t) in enumerate(mgr._reading):
                if tk is self:
                    del mgr._reading[i]
                    if mgr._cancel(self):       # its copy was never handed to the copy stream
                        return
                    if not mgr.out_done(self):
                        mgr._retiring.append((_Parked(self._h, self.policy), t))
                        self._h = None
                        return
                    break
            check(lib().csw_ticket_release(mgr._h, self._h), "csw_ticket_release")
        self._h = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class SwapManager:
    """One per device / replica: pinned pool, staging pool, codec/D2H/H2D streams."""

    def __init__(self, device: Optional[int] = None, pinned_bytes: int = 0, staging_bytes: int = 0,
                 zfp_maxbits: int = 512):
        if device is None:
            device = torch.cuda.current_device()
        self.device = torch.device("cuda", int(device))
        cfg = MgrConfig(int(device), pinned_bytes, staging_bytes, zfp_maxbits)
        h = C.c_void_p()
        with torch.cuda.device(self.device):
            check(lib().csw_mgr_create(C.byref(cfg), C.byref(h)), "csw_mgr_create")
        self._h = h.value
        self.zfp_maxbits = zfp_maxbits
        # Source tensors of swap-outs still being read by the manager's streams.
        # Holding a reference keeps torch's caching allocator from handing the
        # block to someone else; it is dropped at the first call after the
        # device has finished reading.
        self._reading: List[Tuple[Ticket, torch.Tensor]] = []
        # Tickets given up (or whose tensor was taken back) before the copy out had
        # finished, with the tensor they read: released once the device is done
        # with them, never waited for.
        self._retiring: list = []
        self.reclaimed_tensors = 0
        # compressed policies: make the caller's stream wait for the codec's read instead
        # of holding the source tensor until a poll finds the read finished
        self.free_after_codec = True

    def close(self) -> None:
        if self._h is not None:
            check(lib().csw_mgr_destroy(self._h), "csw_mgr_destroy")  # drains the manager's streams
            self._h = None
            self._reading.clear()
            for tk, _ in self._retiring:
                tk._h = None  # the manager and its tickets are gone
            self._retiring.clear()

    def _poll(self) -> None:
        """Drop source tensors the device has finished reading and retire parked
        tickets.  Raw swap-outs finish in order on the copy stream and coded
        ones in order on the codec stream, so each kind is only asked about
        until the first one that is still busy."""
        if self._reading:
            busy = set()
            keep = []
            for tk, t in self._reading:
                if tk._h is None:
                    continue
                kind = tk.policy == POLICY_RAW
                if kind in busy or not self.out_done(tk):
                    busy.add(kind)
                    keep.append((tk, t))
            self._reading = keep
        if self._retiring:
            busy = set()
            keep = []
            for tk, t in self._retiring:
                if tk._h is None:
                    continue
                kind = getattr(tk, "policy", None) == POLICY_RAW
                if kind in busy or not self.out_done(tk):
                    busy.add(kind)
                    keep.append((tk, t))
                else:
                    check(lib().csw_ticket_release(self._h, tk._h), "csw_ticket_release")
                    tk._h = None
            self._retiring = keep

    def reclaim(self, ticket: Ticket) -> Optional[torch.Tensor]:
        """The swapped-out tensor itself, if it has not left yet: while the
        copy out of a losslessly swapped tensor is still queued or running the
        device copy is intact (the manager only reads it), so a consumer that
        needs it now can simply take it back instead of waiting for the copy
        out and a copy in.  The ticket is retired in the background.  None when
        the device copy is gone or the policy is lossy (a lossy swap must hand
        back the decoded values whatever the timing)."""
        if ticket._h is None or ticket.policy not in (POLICY_RAW, POLICY_SPARSE):
            return None
        for i, (tk, t) in enumerate(self._reading):
            if tk is ticket:
                if self.out_done(ticket):
                    return None
                del self._reading[i]
                if not self._cancel(ticket):    # else: never copied at all, nothing to retire
                    self._retiring.append((ticket, t))
                self.reclaimed_tensors += 1
                return t
        return None

    def raw_streams(self) -> Tuple[int, int, int]:
        """(codec, d2h, h2d) cudaStream_t handles of the manager."""
        a, b, c = C.c_void_p(), C.c_void_p(), C.c_void_p()
        check(lib().csw_mgr_get_streams(self._h, C.byref(a), C.byref(b), C.byref(c)), "csw_mgr_get_streams")
        return a.value, b.value, c.value

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_zfp_maxbits(self, maxbits: int) -> None:
        """The reference's setRatio (CSWAP+/Execution.h:63): bits per zfp block."""
        check(lib().csw_mgr_set_zfp_maxbits(self._h, maxbits), "csw_mgr_set_zfp_maxbits")
        self.zfp_maxbits = maxbits

    def keep_staged(self, keep: bool) -> None:
        """Whether a compressed payload stays in device staging after its copy
        out, until the pool needs the room (default), or is released at once."""
        check(lib().csw_mgr_keep_staged(self._h, 1 if keep else 0), "csw_mgr_keep_staged")

    def swap_out(self, t: torch.Tensor, policy: int) -> Ticket:
        _require_cuda_f32(t, "t")
        h = C.c_void_p()
        check(lib().csw_swap_out(self._h, t.data_ptr(), t.numel(), policy, _stream_ptr(t.device), C.byref(h)),
              "csw_swap_out")
        tk = Ticket(self, h.value, t.shape, t.numel(), t.device, policy)
        self._poll()
        if self.free_after_codec and policy in (POLICY_ZFP, POLICY_SPARSE):
            # the codec reads the tensor in a fraction of the time the link needs for it:
            # the caller's stream waits for that read, after which the block may be reused
            # in stream order - no reference is kept, however far the host runs ahead
            self.out_wait(tk)
        else:
            self._reading.append((tk, t))
        return tk

    def import_blob(self, blob, shape=None) -> Ticket:
        """A ticket for a blob made by Ticket.export (here or in another
        process): swap_in() then rebuilds the tensor on this device."""
        import numpy as np
        a = np.ascontiguousarray(np.frombuffer(blob, dtype=np.uint8) if not isinstance(blob, np.ndarray) else blob)
        info = blob_info(a)
        h = C.c_void_p()
        check(lib().csw_blob_import(self._h, a.ctypes.data, a.size, C.byref(h)), "csw_blob_import")
        numel = info["numel"]
        return Ticket(self, h.value, tuple(shape) if shape is not None else (numel,), numel, self.device,
                      info["policy"])

    def _cancel(self, ticket) -> bool:
        """Raw copies out are handed to the copy stream a few at a time; a
        ticket whose copy is still waiting is dropped without ever being
        copied (its handle is dead afterwards)."""
        c = C.c_int()
        check(lib().csw_swap_out_cancel(self._h, ticket._h, C.byref(c)), "csw_swap_out_cancel")
        if c.value:
            ticket._h = None
        return bool(c.value)

    def out_done(self, ticket: Ticket) -> bool:
        d = C.c_int()
        check(lib().csw_swap_out_done(self._h, ticket._h, C.byref(d)), "csw_swap_out_done")
        return bool(d.value)

    def out_wait(self, ticket: Ticket, stream: Optional[torch.cuda.Stream] = None) -> None:
        s = stream.cuda_stream if stream is not None else _stream_ptr(self.device)
        check(lib().csw_swap_out_wait(self._h, ticket._h, s), "csw_swap_out_wait")

    def prefetch(self, ticket: Ticket) -> None:
        check(lib().csw_prefetch(self._h, ticket._h), "csw_prefetch")

    def swap_in(self, ticket: Ticket, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if out is None:
            out = torch.empty(ticket.shape, dtype=torch.float32, device=ticket.device)
        _require_cuda_f32(out, "out")
        if out.numel() != ticket.numel:
            raise ValueError("out has the wrong number of elements")
        check(lib().csw_swap_in(self._h, ticket._h, out.data_ptr(), _stream_ptr(out.device)), "csw_swap_in")
        self._poll()
        return out

    def swap_in_start(self, ticket: Ticket, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """First half of swap_in: copy and decode are enqueued behind the work
        already on the current stream, which is not made to wait.  Call
        swap_in_wait before the tensor is used."""
        if out is None:
            out = torch.empty(ticket.shape, dtype=torch.float32, device=ticket.device)
        _require_cuda_f32(out, "out")
        if out.numel() != ticket.numel:
            raise ValueError("out has the wrong number of elements")
        check(lib().csw_swap_in_start(self._h, ticket._h, out.data_ptr(), _stream_ptr(out.device)),
              "csw_swap_in_start")
        return out

    def swap_in_wait(self, ticket: Ticket) -> None:
        check(lib().csw_swap_in_wait(self._h, ticket._h, _stream_ptr(self.device)), "csw_swap_in_wait")
        self._poll()

    def stats(self) -> dict:
        s = MgrStats()
        check(lib().csw_mgr_get_stats(self._h, C.byref(s)), "csw_mgr_get_stats")
        return {n: getattr(s, n) for n, _ in MgrStats._fields_}

    def reset_stats(self) -> None:
        check(lib().csw_mgr_reset_stats(self._h), "csw_mgr_reset_stats")

    def sync(self) -> None:
        check(lib().csw_mgr_sync(self._h), "csw_mgr_sync")
        self._poll()


@dataclass
class TensorDesc:
    numel: int
    zero_fraction: float = -1.0
    lossy_ok: bool = False
    ready_s: float = 0.0   # forward time at which the swap-out may start
    need_s: float = 0.0    # backward compute that runs before the tensor is needed


_COST_FIELDS = [n for n, _ in CostModelStruct._fields_]


class CostModel:
    """Fitted linear time models of the codecs and the host link, and the
    per-tensor decision raw / sparse / ZFP."""

    def __init__(self, **coeffs):
        self.c = CostModelStruct()
        for k, v in coeffs.items():
            if k not in _COST_FIELDS:
                raise KeyError(k)
            setattr(self.c, k, v)

    @classmethod
    def fit(cls, mgr: SwapManager, zfp_maxbits: Optional[int] = None) -> "CostModel":
        m = cls()
        m.c.zfp_maxbits = zfp_maxbits or mgr.zfp_maxbits
        with torch.cuda.device(mgr.device):
            check(lib().csw_cost_fit(mgr._h, C.byref(m.c)), "csw_cost_fit")
        return m

    def decide(self, tensors: Sequence[TensorDesc], fwd_total_s: float = 0.0) -> Tuple[List[int], List[float]]:
        """Policy code per tensor (forward order) and its modelled stall in seconds."""
        n = len(tensors)
        arr = (TensorDescStruct * max(n, 1))()
        for i, t in enumerate(tensors):
            arr[i] = TensorDescStruct(t.numel, t.zero_fraction, int(t.lossy_ok), t.ready_s, t.need_s)
        pol = (C.c_int * max(n, 1))()
        exp = (C.c_double * max(n, 1))()
        check(lib().csw_cost_decide(C.byref(self.c), arr, n, fwd_total_s, pol, exp), "csw_cost_decide")
        return list(pol[:n]), list(exp[:n])

    def simulate(self, tensors: Sequence[TensorDesc], policy: Sequence[int], fwd_total_s: float = 0.0
                 ) -> Tuple[float, List[float]]:
        """Modelled stall (seconds) of a step that swaps `tensors` under the
        given policy codes: (total, per tensor)."""
        n = len(tensors)
        arr = (TensorDescStruct * max(n, 1))()
        for i, t in enumerate(tensors):
            arr[i] = TensorDescStruct(t.numel, t.zero_fraction, int(t.lossy_ok), t.ready_s, t.need_s)
        pol = (C.c_int * max(n, 1))(*policy)
        exp = (C.c_double * max(n, 1))()
        total = C.c_double()
        check(lib().csw_cost_simulate(C.byref(self.c), arr, n, fwd_total_s, pol, exp, C.byref(total)),
              "csw_cost_simulate")
        return total.value, list(exp[:n])

    def as_dict(self) -> dict:
        return {k: getattr(self.c, k) for k in _COST_FIELDS}

    def save(self, path: str, policy: Optional[Iterable[int]] = None) -> None:
        """Persist the coefficients (and optionally the chosen policy vector)."""
        with open(path, "w") as f:
            json.dump({"cost_model": self.as_dict(), "policy": list(policy) if policy is not None else None}, f,
                      indent=1)

    @classmethod
    def load(cls, path: str) -> Tuple["CostModel", Optional[List[int]]]:
        with open(path) as f:
            d = json.load(f)
        if not isinstance(d, dict) or "cost_model" not in d:
            raise ValueError(f"{path}: not a cost-model file")
        return cls(**d["cost_model"]), d.get("policy")
