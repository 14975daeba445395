"""GPU-resident streaming runtime for exact hard routing.

Host-side mirror of the reference's ``RosaRuntime`` (rosa_soft/runtime.py:311-856, native part
rosa_soft/csrc/rosa_runtime.cpp:216-556) for the 1..8-bit packed deployment subset: same
constructor, properties, ``update`` / ``update_packed`` signatures, slot fixing, ``sequence_ids``
checks, ``reset`` / ``close`` life cycle and error texts.  The difference is where the state
lives: the reference stages every update to the CPU, steps one suffix automaton per
(slot, head) there and copies the result back (runtime.py:728-773); this class keeps the query
and payload histories and one occurrence bitmap per key symbol in HBM and updates them with
``rosa_b200_stream_update`` (a bit-parallel matcher), so a chunk never leaves the device and
the call only enqueues work on a CUDA stream.  Results are identical to a one-shot pass
whatever the chunking.
"""
from __future__ import annotations

import operator
from typing import Any, Dict, Optional, Sequence, Tuple

import torch
from torch import Tensor

from . import cabi

_MIN_CAPACITY = 256


def _as_index(name: str, value) -> int:
    if isinstance(value, bool):
        raise TypeError(f"{name} must be an integer")
    try:
        return operator.index(value)
    except TypeError as error:
        raise TypeError(f"{name} must be an integer") from error


def pack_sign_bits(logits: Tensor) -> Tensor:
    """[..., bits] floating point -> [...] uint8, bit d set iff component d > 0
    (reference runtime.py:130-146)."""
    if not logits.is_floating_point():
        raise TypeError("unpacked RosaRuntime inputs must be floating-point")
    bits = logits.size(-1)
    if not 1 <= bits <= 8:
        raise ValueError(f"RosaRuntime supports 1..8 bits, got {bits}")
    weights = torch.tensor([1 << d for d in range(bits)], dtype=torch.int32, device=logits.device)
    return ((logits > 0).to(torch.int32) * weights).sum(dim=-1).to(torch.uint8).contiguous()


def unpack_sign_bits(packed: Tensor, bits: int, dtype: torch.dtype) -> Tensor:
    """[...] uint8 -> [..., bits] of +-1 (reference runtime.py:149-162)."""
    shifts = torch.arange(bits, dtype=torch.int32, device=packed.device)
    ones = (packed.to(torch.int32).unsqueeze(-1) >> shifts) & 1
    return ones.to(dtype).mul(2).sub(1)


def _sequence_id_tuple(sequence_ids, slot_count: int) -> Optional[Tuple[int, ...]]:
    if sequence_ids is None:
        return None
    if isinstance(sequence_ids, Tensor):
        if sequence_ids.ndim != 1:
            raise ValueError("sequence_ids must be a 1D tensor")
        if sequence_ids.dtype not in (torch.uint8, torch.int8, torch.int16, torch.int32, torch.int64):
            raise TypeError("sequence_ids must contain integers")
        raw = sequence_ids.detach().cpu().tolist()
    elif isinstance(sequence_ids, (str, bytes)) or not isinstance(sequence_ids, Sequence):
        raise TypeError("sequence_ids must be an integer sequence")
    else:
        raw = list(sequence_ids)
    ids = tuple(_as_index("sequence_ids", item) for item in raw)
    if len(ids) != slot_count:
        raise ValueError(f"sequence_ids must contain one ID per slot ({slot_count})")
    if len(set(ids)) != len(ids):
        raise ValueError("sequence_ids must be unique")
    return ids


class RuntimeWork:
    """Handle of an update enqueued with ``async_op=True``: ``wait()`` orders the caller's
    current stream after the update and returns its result (reference runtime.py:242-292)."""

    def __init__(self, result: Tuple[Tensor, Tensor], event: torch.cuda.Event) -> None:
        self._result = result
        self._event = event

    def wait(self) -> Tuple[Tensor, Tensor]:
        device = self._result[1].device
        current = torch.cuda.current_stream(device)
        current.wait_event(self._event)
        for tensor in self._result:
            tensor.record_stream(current)
        return self._result


class RosaRuntime:
    """Packed deployment runtime for exact latest-longest hard routing, state on the GPU.

    Slots are fixed by the first update after construction or ``reset``; supplying
    ``sequence_ids`` on that update enables reorder checks (reference runtime.py:311-318).
    """

    def __init__(self, num_heads: int, num_payload_heads: Optional[int] = None, qk_bits: int = 8,
                 payload_bits: int = 8, max_suffix_length: int = 32) -> None:
        if num_payload_heads is None:
            num_payload_heads = num_heads
        self._num_heads = _as_index("num_heads", num_heads)
        self._num_payload_heads = _as_index("num_payload_heads", num_payload_heads)
        self._qk_bits = _as_index("qk_bits", qk_bits)
        self._payload_bits = _as_index("payload_bits", payload_bits)
        self._max_suffix_length = _as_index("max_suffix_length", max_suffix_length)
        for name, width in (("qk_bits", self._qk_bits), ("payload_bits", self._payload_bits)):
            if not 1 <= width <= 8:
                raise ValueError(
                    f"{name} must be in [1, 8]; RosaRuntime implements only the packed 1..8-bit "
                    "deployment subset of the RosaSoft training contract")
        if self._num_heads < 1 or self._num_payload_heads < 1:
            raise ValueError("num_heads and num_payload_heads must be positive")
        if self._num_heads % self._num_payload_heads != 0:
            raise ValueError("num_heads must be divisible by num_payload_heads")
        if self._max_suffix_length < 1:
            raise ValueError("max_suffix_length must be >= 1")
        cabi.load()  # fail now, not at the first update, when the CUDA library is missing
        self._state = "OPEN"
        self._clear()

    def _clear(self) -> None:
        self._device: Optional[torch.device] = None
        self._slots = -1
        self._capacity = 0
        self._lengths_host: list = []
        self._key_masks: Optional[Tensor] = None       # [slots, H, 2^qk_bits, capacity / 32]
        self._query_history: Optional[Tensor] = None   # [slots, H, capacity]
        self._payload_history: Optional[Tensor] = None  # [slots, Hp, capacity]
        self._lengths: Optional[Tensor] = None
        self._sequence_ids: Optional[Tuple[int, ...]] = None
        self._ids_fixed = False
        self._last_update: Optional[torch.cuda.Event] = None   # orders updates across streams

    # ------------------------------------------------------------------ configuration
    @property
    def num_heads(self) -> int:
        return self._num_heads

    @property
    def num_payload_heads(self) -> int:
        return self._num_payload_heads

    @property
    def qk_bits(self) -> int:
        return self._qk_bits

    @property
    def payload_bits(self) -> int:
        return self._payload_bits

    @property
    def max_suffix_length(self) -> int:
        return self._max_suffix_length

    @property
    def state(self) -> str:
        return self._state

    # ---------------------------------------------------------------------- life cycle
    def _require_open(self) -> None:
        if self._state != "OPEN":
            raise RuntimeError(f"RosaRuntime is {self._state.lower()}")

    def close(self) -> None:
        if self._state == "CLOSED":
            return
        self._clear()
        self._state = "CLOSED"

    def __enter__(self) -> "RosaRuntime":
        self._require_open()
        return self

    def __exit__(self, exc_type, exc, traceback) -> None:
        self.close()

    def reset(self) -> None:
        """Forgets every slot; the next update fixes the slot count again
        (reference rosa_runtime.cpp:492-498, runtime.py:578-588)."""
        self._require_open()
        self._clear()

    def memory_stats(self) -> Dict[str, int]:
        """Counts of what is held.  ``states`` / ``edges`` are zero: there is no automaton; the
        matcher's state is one occurrence bit per key position and symbol
        (reference runtime.py:557-576)."""
        self._require_open()
        tokens = sum(self._lengths_host)
        slots = max(self._slots, 0)
        return {
            "states": 0,
            "edges": 0,
            "payload_symbols": tokens * self._num_payload_heads,
            "automata": slots * self._num_heads,
            "sequences": slots,
            "logical_bytes": tokens * (self._num_heads * (1 + (1 << self._qk_bits) // 8)
                                       + self._num_payload_heads),
            "capacity_tokens": self._capacity,
        }

    def stats(self) -> Tuple[int, int, int]:
        stats = self.memory_stats()
        return stats["states"], stats["edges"], stats["payload_symbols"]

    def state_dict(self) -> Dict[str, Any]:
        """Everything needed to resume the streams on this or another GPU.  (The reference
        declines to checkpoint its automata, runtime.py:590-603; plain arrays have no such
        problem.)"""
        self._require_open()
        used = max(self._lengths_host, default=0)
        config = {name: getattr(self, name) for name in (
            "num_heads", "num_payload_heads", "qk_bits", "payload_bits", "max_suffix_length")}
        state: Dict[str, Any] = {"config": config, "lengths": list(self._lengths_host),
                                 "sequence_ids": self._sequence_ids, "ids_fixed": self._ids_fixed}
        if self._slots > 0:
            state["key_masks"] = self._key_masks[..., :(used + 31) // 32].clone()
            state["query_history"] = self._query_history[..., :used].clone()
            state["payload_history"] = self._payload_history[..., :used].clone()
        return state

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        self._require_open()
        config = {name: getattr(self, name) for name in (
            "num_heads", "num_payload_heads", "qk_bits", "payload_bits", "max_suffix_length")}
        if state_dict["config"] != config:
            raise ValueError("state_dict was produced by a differently configured RosaRuntime")
        self._clear()
        lengths = [int(v) for v in state_dict["lengths"]]
        self._sequence_ids = state_dict.get("sequence_ids")
        self._ids_fixed = bool(state_dict.get("ids_fixed", False))
        if not lengths:
            return
        query_history = state_dict["query_history"]
        if not query_history.is_cuda:
            raise ValueError("state_dict tensors must be CUDA tensors")
        self._device = query_history.device
        self._slots = len(lengths)
        self._lengths_host = lengths
        self._grow(max(lengths))
        used = query_history.shape[-1]
        self._key_masks[..., :(used + 31) // 32] = state_dict["key_masks"]
        self._query_history[..., :used] = query_history
        self._payload_history[..., :used] = state_dict["payload_history"]
        self._lengths.copy_(torch.tensor(lengths, dtype=torch.int32))

    # -------------------------------------------------------------------------- state
    def _grow(self, needed: int) -> None:
        """Makes room for `needed` tokens per slot (capacity doubles; old contents are kept)."""
        if needed <= self._capacity and self._capacity > 0:
            return      # (a first update without tokens still allocates the minimum capacity)
        capacity = max(_MIN_CAPACITY, self._capacity)
        while capacity < needed:
            capacity *= 2
        shape_m = (self._slots, self._num_heads, 1 << self._qk_bits, capacity // 32)
        shape_q = (self._slots, self._num_heads, capacity)
        shape_p = (self._slots, self._num_payload_heads, capacity)
        key_masks = torch.zeros(shape_m, dtype=torch.int32, device=self._device)
        query_history = torch.empty(shape_q, dtype=torch.uint8, device=self._device)
        payload_history = torch.empty(shape_p, dtype=torch.uint8, device=self._device)
        if self._capacity:
            key_masks[..., :self._capacity // 32] = self._key_masks
            query_history[..., :self._capacity] = self._query_history
            payload_history[..., :self._capacity] = self._payload_history
        else:
            self._lengths = torch.zeros(self._slots, dtype=torch.int32, device=self._device)
        self._key_masks, self._query_history, self._payload_history = (
            key_masks, query_history, payload_history)
        self._capacity = capacity

    def _check_sequence_ids(self, sequence_ids: Optional[Tuple[int, ...]]) -> None:
        if not self._ids_fixed:
            self._ids_fixed = True
            self._sequence_ids = sequence_ids
            return
        if self._sequence_ids is None:
            if sequence_ids is not None:
                raise RuntimeError("sequence_ids checking must be enabled on the first update "
                                   "after construction or reset")
            return
        if sequence_ids is None:
            raise RuntimeError("sequence_ids are required because slot checking is enabled")
        if sequence_ids != self._sequence_ids:
            raise RuntimeError("sequence_ids changed; RosaRuntime slots are fixed")

    # ------------------------------------------------------------------------ updates
    def update(self, query_logits: Tensor, key_logits: Tensor, payload_logits: Tensor,
               cu_seqlens: Optional[Tensor] = None, *, stream: Optional[torch.cuda.Stream] = None,
               async_op: bool = False, return_packed: bool = False, sequence_ids=None):
        """Sign-binarises the logits and updates; dense [B, T, H, bits] or, with `cu_seqlens`,
        packed [N, H, bits] (reference runtime.py:605-651)."""
        if query_logits.shape != key_logits.shape:
            raise ValueError(f"query/key shapes differ: {query_logits.shape} vs {key_logits.shape}")
        if query_logits.size(-1) != self.qk_bits:
            raise ValueError("query/key last dimension must equal qk_bits")
        if payload_logits.size(-1) != self.payload_bits:
            raise ValueError("payload last dimension must equal payload_bits")
        rank = 4 if cu_seqlens is None else 3
        if query_logits.ndim != rank or payload_logits.ndim != rank:
            layout = "dense" if cu_seqlens is None else "varlen"
            raise ValueError(f"{layout} inputs have the wrong rank for RosaRuntime")
        return self.update_packed(
            pack_sign_bits(query_logits), pack_sign_bits(key_logits), pack_sign_bits(payload_logits),
            cu_seqlens=cu_seqlens, stream=stream, async_op=async_op, return_packed=return_packed,
            output_dtype=payload_logits.dtype, sequence_ids=sequence_ids)

    def update_packed(self, query_symbols: Tensor, key_symbols: Tensor, payload_symbols: Tensor,
                      cu_seqlens: Optional[Tensor] = None, *,
                      stream: Optional[torch.cuda.Stream] = None, async_op: bool = False,
                      return_packed: bool = True, output_dtype: torch.dtype = torch.float32,
                      sequence_ids=None):
        """Appends one chunk per slot and returns, per chunk token and head, the payload symbol
        that followed the latest-longest match and the matched key end position in the slot's
        whole history (-1 and payload 0 for no match); reference runtime.py:653-789,
        rosa_runtime.cpp:333-482.  Dense chunks are uint8 [B, T, H] / [B, T, Hp]; with
        `cu_seqlens` (int32/int64 [slots + 1]) they are packed [N, H] / [N, Hp]."""
        tensors = (query_symbols, key_symbols, payload_symbols)
        if any(t.dtype != torch.uint8 for t in tensors):
            raise TypeError("packed RosaRuntime inputs must have dtype torch.uint8")
        if query_symbols.shape != key_symbols.shape:
            raise ValueError("packed query/key shapes differ: "
                             f"{query_symbols.shape} vs {key_symbols.shape}")
        if not query_symbols.device == key_symbols.device == payload_symbols.device:
            raise ValueError("all packed inputs must be on the same device")
        dense = cu_seqlens is None
        if dense:
            if query_symbols.ndim != 3 or payload_symbols.ndim != 3:
                raise ValueError("dense packed inputs must have shapes [B, T, H] and [B, T, H_v]")
            if query_symbols.shape[:2] != payload_symbols.shape[:2]:
                raise ValueError("dense query and payload dimensions B,T must match")
            slots, tokens = query_symbols.shape[:2]
            if slots < 1:
                raise ValueError("dense batch size must be >= 1")
            offsets = [s * tokens for s in range(slots + 1)]
        else:
            if query_symbols.ndim != 2 or payload_symbols.ndim != 2:
                raise ValueError("varlen packed inputs must have shapes [total, H] and [total, H_v]")
            if query_symbols.size(0) != payload_symbols.size(0):
                raise ValueError("varlen query and payload token counts must match")
            if cu_seqlens.ndim != 1:
                raise ValueError("cu_seqlens must be a 1D tensor")
            if cu_seqlens.numel() < 2:
                raise ValueError("cu_seqlens must describe at least one sequence")
            if cu_seqlens.dtype not in (torch.int32, torch.int64):
                raise TypeError("cu_seqlens must have dtype int32 or int64")
            offsets = [int(v) for v in cu_seqlens.detach().cpu().tolist()]
            slots = len(offsets) - 1
            if offsets[0] != 0:
                raise ValueError("cu_seqlens must start at 0")
            if any(b < a for a, b in zip(offsets, offsets[1:])):
                raise ValueError("cu_seqlens must be non-decreasing")
            if offsets[-1] != query_symbols.size(0):
                raise ValueError("cu_seqlens[-1] must equal the total token count")
        heads, payload_heads = query_symbols.shape[-1], payload_symbols.shape[-1]
        if heads != self.num_heads:
            raise ValueError("packed query/key head count must equal num_heads")
        if payload_heads != self.num_payload_heads:
            raise ValueError("packed payload head count must equal num_payload_heads")
        ids = _sequence_id_tuple(sequence_ids, slots)
        device = query_symbols.device
        if not query_symbols.is_cuda:
            raise ValueError("rosa_soft_b200.RosaRuntime keeps its state on the GPU: inputs must "
                             "be CUDA tensors")
        if stream is not None and stream.device != device:
            raise ValueError("stream and inputs must use the same CUDA device")
        if not return_packed and not torch.empty((), dtype=output_dtype).is_floating_point():
            raise TypeError("output_dtype must be floating-point when unpacking")
        self._require_open()

        if self._slots == -1:
            self._slots, self._device = slots, device
            self._lengths_host = [0] * slots
        elif slots != self._slots:
            raise RuntimeError("RosaRuntime slot count is fixed after the first update")
        elif device != self._device:
            raise ValueError("RosaRuntime state lives on another device")
        self._check_sequence_ids(ids)

        chunk = [b - a for a, b in zip(offsets, offsets[1:])]
        after = [held + n for held, n in zip(self._lengths_host, chunk)]
        if max(after) > 2**31 - 1:
            raise RuntimeError("ROSA sequence length exceeded int32 range")
        current = torch.cuda.current_stream(device)
        run_on = stream if stream is not None else current
        if stream is not None:
            stream.wait_stream(current)   # the inputs were produced on the caller's stream
        if self._last_update is not None:
            # the state is shared by all updates: whatever stream the previous one ran on, this
            # one starts after it (the C ABI wants calls that share a state ordered)
            run_on.wait_event(self._last_update)
        with torch.cuda.stream(run_on):
            self._grow(max(after))
            flat_q = query_symbols.reshape(-1, heads).contiguous()
            flat_k = key_symbols.reshape(-1, heads).contiguous()
            flat_p = payload_symbols.reshape(-1, payload_heads).contiguous()
            dev_offsets = torch.tensor(offsets, dtype=torch.int32).to(device, non_blocking=True)
            packed, end, workspace = cabi.stream_update(
                flat_q, flat_k, flat_p, dev_offsets, self.qk_bits, self.payload_bits,
                self.max_suffix_length, self._key_masks, self._query_history, self._payload_history,
                self._lengths, max(after), stream=run_on.cuda_stream)
            self._lengths_host = after
            if dense:
                packed = packed.reshape(slots, tokens, heads)
                end = end.reshape(slots, tokens, heads)
            if return_packed:
                result = (packed, end)
            else:
                values = unpack_sign_bits(packed, self.payload_bits, output_dtype)
                values = torch.where(end.unsqueeze(-1) >= 0, values,
                                     torch.zeros((), dtype=output_dtype, device=device))
                result = (values, end)
            for tensor in (flat_q, flat_k, flat_p, dev_offsets, workspace, self._key_masks,
                           self._query_history, self._payload_history, self._lengths):
                tensor.record_stream(run_on)
            self._last_update = torch.cuda.Event()
            self._last_update.record(run_on)
        if stream is None:
            if async_op:
                event = torch.cuda.Event()
                event.record(current)
                return RuntimeWork(result, event)
            return result
        event = torch.cuda.Event()
        event.record(stream)
        work = RuntimeWork(result, event)
        return work if async_op else work.wait()
