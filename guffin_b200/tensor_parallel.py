"""Optional tensor parallelism for one stream's latency: G shards (one per GPU) each hold 1 / G of every
matrix of one model and run the same passes; the partial sums behind the O and down projections are summed
across the shards inside the projection launches over peer memory (gf_model_shard_*), or by a host reduction
hook (gf_model_set_reduce_hook: NCCL, or an in-process sum).  The reference runs on one device and has no
counterpart; the single-GPU plan stays the product path and the parity anchor, and this mode is checked
against it.

Sharding (GGUF matrices are [K inputs] x [N output columns], stored column after column, each column K / block
native blocks):
  attn_q, attn_k, attn_v   by output column: whole heads, heads / G (kv_heads / G) per shard
  attn_output              by input row: the K slice fed by the shard's own heads
  ffn_gate, ffn_up         by output column: ffn / G per shard
  ffn_down                 by input row: the K slice fed by the shard's own gate/up columns
  output (the head)        by output column: vocab / G per shard; an F16 or tied table is sliced the same way
  token_embd               whole (a gather of one row per token; gf_model_set_token_table_vocab)
  norms                    whole
A shard's plan is an ordinary plan on the local geometry, so every kernel, graph and KV ring is the
single-GPU one at 1 / G of the width.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import synthetic as syn
from .lib import check, load
from .model import CandidateResult, Model

REDUCE_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p)

_BLOCK = {syn.Q8_0: (32, 34), syn.Q4_K: (256, 144), syn.Q6_K: (256, 210), 1: (1, 2)}      # elements, bytes (1 = F16)


def shard_config(config: dict, size: int) -> dict:
    """The local geometry of one of `size` shards."""
    for key in ("heads", "kv_heads", "ffn", "vocab"):
        if config[key] % size:
            raise ValueError(f"{key} = {config[key]} does not divide into {size} shards")
    if (config["ffn"] // size) % 256 or (config["vocab"] // size) % 8:
        raise ValueError("a shard's FFN slice must be a multiple of 256 and its vocabulary slice of 8")
    local = dict(config)
    for key in ("heads", "kv_heads", "ffn", "vocab"):
        local[key] = config[key] // size
    return local


def _columns(value, rank: int, size: int):
    """Output columns [rank * N / size, (rank + 1) * N / size) of a native matrix."""
    dtype, k, n, data = value[:4]
    elements, block_bytes = _BLOCK[dtype]
    column_bytes = k // elements * block_bytes
    local = n // size
    raw = np.ascontiguousarray(data).view(np.uint8).reshape(n, column_bytes)
    return (dtype, k, local, np.ascontiguousarray(raw[rank * local:(rank + 1) * local]).reshape(-1)) + tuple(value[4:])


def _rows(value, rank: int, size: int):
    """Input rows [rank * K / size, (rank + 1) * K / size) of every column of a native matrix."""
    dtype, k, n, data = value[:4]
    elements, block_bytes = _BLOCK[dtype]
    local = k // size
    if local % elements:
        raise ValueError("a K slice must hold whole blocks")
    blocks, local_blocks = k // elements, local // elements
    raw = np.ascontiguousarray(data).view(np.uint8).reshape(n, blocks, block_bytes)
    return (dtype, local, n, np.ascontiguousarray(raw[:, rank * local_blocks:(rank + 1) * local_blocks]).reshape(-1)) + tuple(value[4:])


def shard_weights(weights, rank: int, size: int):
    """(name, value) pairs of shard `rank`, from the full model's pairs (a dict or any iterable, such as
    synthetic.iter_model_weights: one full tensor is alive at a time).  A model whose head is tied to the
    token table gets an explicit `output.weight` slice of that table."""
    has_head = False
    table = None
    for name, value in (weights.items() if hasattr(weights, "items") else weights):
        short = name.split(".")[2] if name.startswith("blk.") else name.split(".")[0]
        if not isinstance(value, tuple):
            yield name, value
        elif short in ("attn_q", "attn_k", "attn_v", "ffn_gate", "ffn_up"):
            yield name, _columns(value, rank, size)
        elif short in ("attn_output", "ffn_down"):
            yield name, _rows(value, rank, size)
        elif short == "output":
            has_head = True
            yield name, _columns(value, rank, size)
        elif short == "token_embd":
            table = value
            yield name, value
        else:
            raise KeyError(name)
    if not has_head:
        if table is None:
            raise ValueError("no token table to cut the head from")
        yield "output.weight", _columns(table, rank, size)


class Shard:
    """One shard's plan.  The partial sums behind O and down are summed either
      * inside the projection launches over peer memory (reduce=None, the default): call `exported()` /
        `arena` on every shard, then `connect_exported(handles)` (shards in different processes) or
        `connect(arenas)` (one process, one GPU per shard) on every shard, then a host barrier; or
      * by a host hook: `reduce` is a (function pointer, user pointer) pair for gf_model_set_reduce_hook --
        REDUCE_FN(python_callable) for an in-process sum, or (libguffin_tp.gf_tp_reduce, communicator)."""

    def __init__(self, config: dict, weights, context: int, rank: int, size: int, reduce=None, row_capacity: int = 2):
        self.rank, self.size = rank, size
        self.full_vocab = config["vocab"]
        self.local_vocab = config["vocab"] // size
        self._reduce = reduce           # keeps a ctypes callback alive as long as the plan

        def before_binding(model):
            check(model.L.gf_model_set_token_table_vocab(model.handle, self.full_vocab))
            if reduce is not None:
                function, user = reduce
                check(model.L.gf_model_set_reduce_hook(model.handle, C.cast(function, C.c_void_p), user))

        self.model = Model(shard_config(config, size), shard_weights(weights, rank, size), context, row_capacity,
                           before_binding=before_binding)
        self._handle = None
        if reduce is None:
            handle = C.create_string_buffer(64)
            check(self.model.L.gf_model_shard_prepare(self.model.handle, rank, size, handle))
            self._handle = handle.raw

    def exported(self) -> bytes:
        """The 64-byte handle other processes map this shard's arena with."""
        return self._handle

    @property
    def arena(self) -> int:
        return self.model.L.gf_model_shard_arena(self.model.handle)

    def connect(self, arenas) -> None:
        table = (C.c_void_p * self.size)(*arenas)
        check(self.model.L.gf_model_shard_connect(self.model.handle, table))

    def connect_exported(self, handles) -> None:
        blob = b"".join(handles)
        assert len(blob) == 64 * self.size
        check(self.model.L.gf_model_shard_connect_ipc(self.model.handle, blob))

    def global_selection(self, enable: bool = True) -> None:
        """select / read_candidates in ids of the whole vocabulary, merged over the shards (for an H1 engine per
        shard running in step)."""
        check(self.model.L.gf_model_shard_global_selection(self.model.handle, int(enable)))

    def global_candidates(self, result: CandidateResult) -> np.ndarray:
        """A shard's candidates with ids moved into the full vocabulary."""
        pairs = result.pairs()
        pairs["token"] += np.uint32(self.rank * self.local_vocab)
        return pairs


def merge_candidates(per_shard: list, retain: int) -> np.ndarray:
    """The full model's candidate list from the shards' lists (ids already global): the `retain` largest
    logits, ties broken by the smaller id -- the order gf_token_candidates itself returns
    (select_candidates, src/tensor/backends/metal/token_candidates.cpp)."""
    pairs = np.concatenate(per_shard)
    order = np.lexsort((pairs["token"], -pairs["logit"].astype(np.float64)))
    return pairs[order[:retain]]


class NcclReducer:
    """The NCCL all-reduce hook of libguffin_tp.so for one process of `size`; `exchange(bytes_or_None) -> bytes`
    hands rank 0's 128-byte id to every rank (a torch.distributed broadcast in the bench)."""

    def __init__(self, rank: int, size: int, exchange):
        import os
        from . import build
        path = build.build_tp()
        if path is None or not os.path.exists(path):
            raise RuntimeError("libguffin_tp.so is not built (NCCL header or library missing)")
        load()                          # the device is chosen by the caller before this point
        self.lib = C.CDLL(path)
        self.lib.gf_tp_unique_id.argtypes = [C.c_void_p]
        self.lib.gf_tp_create.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_void_p)]
        self.lib.gf_tp_destroy.argtypes = [C.c_void_p]
        ident = C.create_string_buffer(128)
        if rank == 0:
            check(self.lib.gf_tp_unique_id(ident))
        ident = C.create_string_buffer(exchange(ident.raw if rank == 0 else None), 128)
        self.comm = C.c_void_p()
        check(self.lib.gf_tp_create(ident, rank, size, C.byref(self.comm)))
        self.hook = (self.lib.gf_tp_reduce, self.comm)

    def close(self):
        if self.comm:
            self.lib.gf_tp_destroy(self.comm)
            self.comm = C.c_void_p()


class ThreadReducer:
    """An in-process reduction for shards that live on ONE device, each driven by its own host thread (plans
    with CUDA graphs off: the hook synchronises).  Every shard copies its buffer into its slot, all meet at a
    barrier, and each sums the slots in rank order, so every shard holds the same bits.  A way to check the
    sharded arithmetic where a single GPU is at hand; the multi-GPU path is NcclReducer."""

    def __init__(self, size: int, max_count: int):
        import threading
        from .lib import DeviceBuffer
        self.size = size
        self.max_count = max_count
        self.slots = [DeviceBuffer(max_count * 4) for _ in range(size)]
        self.barrier = threading.Barrier(size)
        self.calls = 0

    def hook(self, rank: int):
        L = load()

        def reduce(user, buffer, count, stream):
            try:
                if count > self.max_count:
                    return -1
                check(L.gf_copy(self.slots[rank].ptr, buffer, count * 4, stream))
                check(L.gf_stream_synchronize(stream))
                self.barrier.wait(timeout=60)
                if self.size > 1:                       # size 1: the buffer already holds the sum
                    check(L.gf_add(self.slots[0].ptr, self.slots[1].ptr, buffer, count, stream))
                for other in range(2, self.size):
                    check(L.gf_add(buffer, self.slots[other].ptr, buffer, count, stream))
                check(L.gf_stream_synchronize(stream))
                self.barrier.wait(timeout=60)           # no slot is overwritten before every shard has read it
                if rank == 0:
                    self.calls += 1
                return 0
            except Exception:
                self.barrier.abort()
                return -3

        return (REDUCE_FN(reduce), None)
