"""Tensor parallelism on the host side (no counterpart in the reference, which runs on one CPU).

One process per GPU.  Every rank builds `LanguageModel(config, tokenizer, weights, tp_size=g, tp_rank=r)` from the FULL
weights; the library keeps the rank's shard.  `connect(model, group)` then moves the exchange-memory handles between
the ranks (torch.distributed, any backend) and wires the peers.  After that, `transformer_`, `generate` and `sample`
are called by all ranks with the same arguments and return the same result on every rank.

The partition (heads by kv group, ffn by hidden units, wo and w2 by super-block columns of their input) is stated
once more here in numpy, `shard_weights`, so that it can be checked against the CPU oracle without a GPU:
the sum over ranks of the sharded layer equals the unsharded layer.
"""
import ctypes as C
from typing import List

import numpy as np

from . import _lib as L
from .model import LanguageModel, ModelConfig, QuantMatrix, TransformerLayerWeights, TransformerWeights


def check_shardable(c: ModelConfig, tp_size: int) -> None:
    if tp_size < 1 or tp_size > 8:
        raise ValueError("tp_size must be in 1..8")
    if c.n_kv_heads % tp_size:
        raise ValueError("n_kv_heads must be a multiple of tp_size")
    if (c.dim // tp_size) % 256 or (c.hidden_dim // tp_size) % 256 or c.hidden_dim % tp_size:
        raise ValueError("dim / tp_size and hidden_dim / tp_size must be multiples of 256")


def shard_plan(c: ModelConfig, tp_size: int, rank: int) -> dict:
    """Row / block-column ranges rank `rank` keeps.  Rows are output rows of the matrix; block columns are
    256-value super-blocks of its input."""
    check_shardable(c, tp_size)
    hs = c.dim // c.n_heads
    lh, lkv, lhid = c.n_heads // tp_size, c.n_kv_heads // tp_size, c.hidden_dim // tp_size
    nb_o, nb_2 = c.dim // 256 // tp_size, lhid // 256
    return {
        "n_heads": lh, "n_kv_heads": lkv, "hidden_dim": lhid,
        "wq_rows": (rank * lh * hs, (rank + 1) * lh * hs),
        "wk_rows": (rank * lkv * hs, (rank + 1) * lkv * hs),
        "wv_rows": (rank * lkv * hs, (rank + 1) * lkv * hs),
        "w1_rows": (rank * lhid, (rank + 1) * lhid),
        "w3_rows": (rank * lhid, (rank + 1) * lhid),
        "wo_block_cols": (rank * nb_o, (rank + 1) * nb_o),
        "w2_block_cols": (rank * nb_2, (rank + 1) * nb_2),
    }


def _rows(a, lo, hi):
    return a.rows(lo, hi) if isinstance(a, QuantMatrix) else np.ascontiguousarray(a[lo:hi])


def _block_cols(a: QuantMatrix, lo, hi) -> QuantMatrix:
    if not isinstance(a, QuantMatrix):
        raise L.L2BError(L.ERR_UNSUPPORTED_TYPE, "tensor parallelism needs k-quant wo and w2 matrices")
    bb = L.BLOCK_BYTES[a.ggml_type]
    nb = a.in_dim // 256
    d = np.asarray(a.data).reshape(a.out_dim, nb, bb)[:, lo:hi, :]
    return QuantMatrix(a.ggml_type, np.ascontiguousarray(d).reshape(-1), (hi - lo) * 256, a.out_dim)


def shard_weights(c: ModelConfig, w: TransformerWeights, tp_size: int, rank: int) -> TransformerWeights:
    """The shard of rank `rank` as plain arrays (what the library keeps after l2b_model_upload_tensor)."""
    pl = shard_plan(c, tp_size, rank)
    layers = [TransformerLayerWeights(
        lw.rms_att_weight, lw.rms_ffn_weight,
        _rows(lw.wq, *pl["wq_rows"]), _rows(lw.wk, *pl["wk_rows"]), _rows(lw.wv, *pl["wv_rows"]),
        _block_cols(lw.wo, *pl["wo_block_cols"]),
        _rows(lw.w1, *pl["w1_rows"]), _block_cols(lw.w2, *pl["w2_block_cols"]), _rows(lw.w3, *pl["w3_rows"]))
        for lw in w.layers]
    return TransformerWeights(w.token_embedding_table, layers, w.rms_final_weight, w.output_weight)


def exchange_handles(handle: bytes, group=None) -> List[bytes]:
    """All ranks' 64-byte handles, ordered by rank (torch.distributed all_gather_object; gloo or nccl)."""
    import torch.distributed as dist

    n = dist.get_world_size(group)
    out = [None] * n
    dist.all_gather_object(out, bytes(handle), group=group)
    if any(h is None or len(h) != 64 for h in out):
        raise RuntimeError("handle exchange failed")
    return out


def connect(model: LanguageModel, group=None) -> None:
    """Wire the ranks of a tensor-parallel model: export this rank's handle, gather all, map the peers."""
    import torch.distributed as dist

    dev = model.device_model()
    lib = L.lib()
    h = C.create_string_buffer(64)
    L.check(lib.l2b_session_tp_handle(dev.session, h))
    handles = exchange_handles(h.raw, group)
    blob = C.create_string_buffer(b"".join(handles), 64 * len(handles))
    L.check(lib.l2b_session_tp_connect(dev.session, blob, len(handles)))
    dist.barrier(group)  # nobody starts a token before every rank is wired
