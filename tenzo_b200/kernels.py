"""Per-kernel Python entry points over include/tenzo_kernels.h.

torch is used for device memory and the current stream only; every function is exactly one call
through the C ABI into libtenzo_runtime.so and raises if that call reports an error. There is no
eager/PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import abi, load_library

EPI_STORE, EPI_RESIDUAL, EPI_RELU2_GLU = 0, 1, 2


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    if t is None:
        return None
    assert t.is_cuda and t.is_contiguous()
    return t.data_ptr()


def _rows(t: torch.Tensor | None) -> int | None:
    """Pointer of a 2-D tensor whose rows are contiguous but may be strided (a column slice of a wider buffer)."""
    if t is None:
        return None
    assert t.is_cuda and t.dim() == 2 and t.stride(1) == 1
    return t.data_ptr()


def _ok(rc: int, what: str):
    if rc != 0:
        raise RuntimeError(f"{what} failed: rc={rc}" + (f" ({torch.cuda.get_device_name()})" if rc > 0 else " (bad arguments)"))


def tl1_gemv(x: torch.Tensor, w: torch.Tensor, n_blocks: int, K: int, scales, seg_ends=None, *, epilogue=EPI_STORE,
             resid=None, norm_w=None, do_norm=False, eps=1e-5, want_acc=False, want_act=False, use_pdl=False, out=None, prefetch=None,
             workspace=None):
    """x [batch, K] fp32, w TL1-packed uint8. Returns dict(out=..., acc=..., a=..., inv=...)."""
    lib = load_library()
    batch = x.shape[0]
    n_out = n_blocks * 64 // (2 if epilogue == EPI_RELU2_GLU else 1)
    if out is None:
        out = torch.empty(batch, n_out, dtype=torch.float32, device=x.device)
    acc = torch.empty(batch, n_blocks * 64, dtype=torch.int32, device=x.device) if want_acc else None
    a8 = torch.empty(batch, K, dtype=torch.int8, device=x.device) if want_act else None
    inv = torch.empty(batch, dtype=torch.float32, device=x.device) if want_act else None
    scales = list(scales) + [0.0] * (3 - len(scales))
    seg_ends = list(seg_ends) if seg_ends is not None else [n_blocks] * 3
    seg_ends = seg_ends + [n_blocks] * (3 - len(seg_ends))
    g = abi.Tl1GemvArgs()
    g.x, g.norm_w, g.do_norm, g.eps = _ptr(x), _ptr(norm_w), int(do_norm), eps
    g.w, g.n_blocks, g.K = _ptr(w), n_blocks, K
    g.seg_end = (C.c_int * 3)(*seg_ends)
    g.seg_scale = (C.c_float * 3)(*scales)
    g.epilogue, g.resid, g.out = epilogue, _ptr(resid), _ptr(out)
    g.acc_out, g.a_out, g.inv_out = _ptr(acc), _ptr(a8), _ptr(inv)
    g.batch, g.x_stride, g.out_stride = batch, x.stride(0), out.stride(0)
    ws = workspace
    if batch > 1 and ws is None:
        ws = torch.empty(lib.tenzo_cuda_tl1_gemv_workspace_bytes(batch, K), dtype=torch.uint8, device=x.device)
    g.workspace, g.use_pdl = _ptr(ws), int(use_pdl)
    if prefetch is not None:
        g.prefetch, g.prefetch_bytes = _ptr(prefetch), prefetch.numel() * prefetch.element_size()
    _ok(lib.tenzo_cuda_tl1_gemv(C.byref(g), _stream()), "tenzo_cuda_tl1_gemv")
    return dict(out=out, acc=acc, a=a8, inv=inv)


def rmsnorm_quant(x: torch.Tensor, norm_w=None, *, do_norm=True, eps=1e-5, qmax=31, want_y=True, want_q=True):
    lib = load_library()
    batch, dim = x.shape
    y = torch.empty_like(x) if want_y else None
    q = torch.empty(batch, dim, dtype=torch.int8, device=x.device) if want_q else None
    s = torch.empty(batch, dtype=torch.float32, device=x.device) if want_q else None
    _ok(lib.tenzo_cuda_rmsnorm_quant(_ptr(x), _ptr(norm_w), int(do_norm), eps, dim, qmax, batch, x.stride(0), _ptr(y),
                                     _ptr(q), _ptr(s), _stream()), "tenzo_cuda_rmsnorm_quant")
    return y, q, s


def attention_workspace_bytes(batch, n_q, n_kv, max_len) -> int:
    lib = load_library()
    lib.tenzo_cuda_attention_workspace_bytes.restype = C.c_size_t
    lib.tenzo_cuda_attention_workspace_bytes.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int]
    return int(lib.tenzo_cuda_attention_workspace_bytes(batch, n_q, n_kv, max_len))


def attention_int8(q, k, v, cache_k, cache_v, scale_k, scale_v, pos, *, layer, n_q, n_kv, max_seq, rope_cos=None,
                   rope_sin=None, append=True, max_len=None, use_pdl=False, heads_per_cta=0, out=None, tiles=0,
                   block_table=None, n_layers=0, mode=0, split_keys=0, workspace=None):
    """q [batch, n_q*128], k/v [batch, n_kv*128]; caches [batch, layers, n_kv, max_seq, 128] int8 and
    [batch, layers, n_kv, max_seq] fp32; pos int32 [batch]. Returns out [batch, n_q*128].
    With block_table (int32 [batch, blocks per sequence]) the caches are the paged_int8 pools
    [blocks, n_layers, n_kv, 16, 128] / [blocks, n_layers, n_kv, 16] and the arithmetic is the paged cache's."""
    lib = load_library()
    batch = q.shape[0]
    if max_len is None:
        max_len = int(pos.max().item()) + 1
    if out is None:
        out = torch.empty(batch, n_q * 128, dtype=torch.float32, device=q.device)
    a = abi.AttentionArgs()
    a.q, a.k, a.v, a.out = _rows(q), _rows(k), _rows(v), _ptr(out)
    a.q_stride, a.kv_stride = q.stride(0), (k.stride(0) if k is not None else 0)
    a.cache_k, a.cache_v, a.scale_k, a.scale_v = _ptr(cache_k), _ptr(cache_v), _ptr(scale_k), _ptr(scale_v)
    a.seq_stride_kv, a.seq_stride_sc = cache_k.stride(0), scale_k.stride(0)
    a.pos, a.rope_cos, a.rope_sin = _ptr(pos), _ptr(rope_cos), _ptr(rope_sin)
    a.layer, a.n_q, a.n_kv, a.head_dim, a.max_seq = layer, n_q, n_kv, 128, max_seq
    a.batch, a.max_len, a.append, a.use_pdl, a.heads_per_cta = batch, max_len, int(append), int(use_pdl), heads_per_cta
    a.tiles = tiles
    if block_table is not None:
        assert block_table.dtype == torch.int32 and block_table.is_contiguous()
        a.block_table, a.table_stride, a.n_layers = _ptr(block_table), (block_table.stride(0) if block_table.dim() == 2 else 0), n_layers
        a.n_pool_blocks = cache_k.shape[0]
    if mode == 1:
        if workspace is None:
            workspace = torch.empty(attention_workspace_bytes(batch, n_q, n_kv, max_len), dtype=torch.uint8, device=q.device)
        a.mode, a.split_keys, a.workspace, a.workspace_bytes = 1, split_keys, _ptr(workspace), workspace.numel()
    _ok(lib.tenzo_cuda_attention_int8(C.byref(a), _stream()), "tenzo_cuda_attention_int8")
    return out


def lm_head_i8(x, w, row_scales, *, norm_w=None, do_norm=True, eps=1e-5, want_logits=True, want_acc=False, use_pdl=False, logits=None):
    lib = load_library()
    batch, hidden = x.shape
    vocab = w.shape[0]
    if logits is None and want_logits:
        logits = torch.empty(batch, vocab, dtype=torch.float32, device=x.device)
    acc = torch.empty(batch, vocab, dtype=torch.int32, device=x.device) if want_acc else None
    arg = torch.empty(batch, dtype=torch.int32, device=x.device)
    scratch = torch.empty(lib.tenzo_cuda_lm_head_scratch_bytes(batch), dtype=torch.uint8, device=x.device)
    _ok(lib.tenzo_cuda_lm_head_i8(_ptr(x), _ptr(norm_w), int(do_norm), eps, _ptr(w), _ptr(row_scales), vocab, hidden,
                                  batch, x.stride(0), _ptr(logits), _ptr(acc), _ptr(arg), _ptr(scratch), int(use_pdl),
                                  _stream()), "tenzo_cuda_lm_head_i8")
    return logits, acc, arg


def lm_head_i8_static(x, w, row_scales, *, norm_w=None, do_norm=True, eps=1e-5, logits=None, argmax=None, use_pdl=False):
    """LM head through the allocation-free entry point: the caller passes every buffer (logits
    [batch, vocab] fp32 and argmax [batch] int32, both preallocated); the library allocates nothing."""
    lib = load_library()
    batch, hidden = x.shape
    _ok(lib.tenzo_cuda_lm_head_i8_static(_ptr(x), _ptr(norm_w), int(do_norm), eps, _ptr(w), _ptr(row_scales), w.shape[0],
                                         hidden, batch, x.stride(0), _ptr(logits), None, _ptr(argmax), int(use_pdl), _stream()),
        "tenzo_cuda_lm_head_i8_static")
    return logits, argmax


def embedding_i8(w, row_scales, tokens):
    lib = load_library()
    batch, hidden = tokens.shape[0], w.shape[1]
    x = torch.empty(batch, hidden, dtype=torch.float32, device=w.device)
    _ok(lib.tenzo_cuda_embedding_i8(_ptr(w), _ptr(row_scales), hidden, _ptr(tokens), batch, _ptr(x), hidden, w.shape[0], _stream()),
        "tenzo_cuda_embedding_i8")
    return x


def tl1_pack_rows2bit(raw, N, K):
    lib = load_library()
    packed = torch.empty(N * K // 4, dtype=torch.uint8, device=raw.device)
    _ok(lib.tenzo_cuda_tl1_pack_rows2bit(_ptr(raw), N, K, _ptr(packed), _stream()), "tenzo_cuda_tl1_pack_rows2bit")
    return packed
