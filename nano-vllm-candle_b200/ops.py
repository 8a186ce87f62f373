"""Kernel-level Python entry points: torch tensors are used ONLY as device-memory handles
(data_ptr) and for the current CUDA stream; all compute is in libnvc_b200.so through the C ABI
(include/nvc_b200.h).  There is no torch / CPU fallback: a missing library or a non-zero status
raises."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from ._lib import check

BF16 = torch.bfloat16


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _req(t: torch.Tensor, dtype, name: str):
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (no CPU fallback on this path)")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")


class Context:
    """nvc_ctx: one per (process, device).  Mirrors TPConfig{size, rank} (src/tp.rs:3-70)."""

    def __init__(self, device: int = 0, tp_rank: int = 0, tp_size: int = 1):
        self.l = _lib.lib()
        h = C.c_void_p()
        check(self.l.nvc_ctx_create(device, tp_rank, tp_size, C.byref(h)), "nvc_ctx_create")
        self.h = h
        self.device = device
        self.tp_rank, self.tp_size = tp_rank, tp_size
        self.num_sms = self.l.nvc_ctx_num_sms(self.h)
        self._ws = None

    def close(self):
        if self.h:
            self.l.nvc_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _ck(self, st, where):
        check(st, where, self.h)

    # ---- collectives
    @staticmethod
    def nccl_unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        check(_lib.lib().nvc_nccl_unique_id(buf), "nvc_nccl_unique_id")
        return buf.raw

    def init_nccl(self, unique_id: bytes):
        assert len(unique_id) == 128
        self._ck(self.l.nvc_ctx_init_nccl(self.h, C.c_char_p(unique_id)), "nvc_ctx_init_nccl")

    def p2p_export(self, slot_bytes: int) -> bytes:
        """Allocates this rank's peer buffer; returns the 64-byte CUDA IPC handle to all-gather."""
        buf = C.create_string_buffer(64)
        self._ck(self.l.nvc_ctx_p2p_export(self.h, slot_bytes, buf), "nvc_ctx_p2p_export")
        return buf.raw

    def p2p_import(self, handles) -> None:
        """handles: the tp_size 64-byte handles in rank order."""
        blob = b"".join(handles)
        assert len(blob) == 64 * self.tp_size
        self._ck(self.l.nvc_ctx_p2p_import(self.h, C.c_char_p(blob)), "nvc_ctx_p2p_import")

    def init_tp(self, dist, slot_bytes: int = 4 << 20) -> None:
        """NCCL communicator + NVLink peer buffers, rendezvous through torch.distributed."""
        box = [Context.nccl_unique_id() if self.tp_rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        self.init_nccl(box[0])
        mine = self.p2p_export(slot_bytes)
        allh = [None] * self.tp_size
        dist.all_gather_object(allh, mine)
        self.p2p_import(allh)

    def nvls_init(self, slot_bytes: int, ll_buf_bytes: int = 4 << 20, group_name: Optional[str] = None) -> bool:
        """COLLECTIVE: the NVSwitch multicast buffers of the TP group (nvc_ctx_nvls_init).  False (on every rank
        alike) when multicast is not available on this box; nvls_status() then says why."""
        st = self.l.nvc_ctx_nvls_init(self.h, slot_bytes, ll_buf_bytes, None if group_name is None else group_name.encode())
        if st == -8:
            return False
        self._ck(st, "nvc_ctx_nvls_init")
        return True

    def nvls_ready(self) -> bool:
        return bool(self.l.nvc_ctx_nvls_ready(self.h))

    def nvls_status(self) -> str:
        return self.l.nvc_ctx_nvls_status(self.h).decode()

    def nvls_slot(self, rows: int, cols: int) -> torch.Tensor:
        """This rank's NVLS slot viewed as a bf16 [rows, cols] tensor (memory owned by the context)."""
        nbytes = rows * cols * 2
        assert nbytes <= self.l.nvc_ctx_nvls_slot_bytes(self.h)
        ptr = self.l.nvc_ctx_nvls_slot(self.h)
        iface = {"shape": (rows, cols), "typestr": "<u2", "data": (ptr, False), "version": 3}
        holder = type("_Slot", (), {"__cuda_array_interface__": iface})()
        return torch.as_tensor(holder, device=f"cuda:{self.device}").view(BF16)

    def nvls_allreduce_rmsnorm(self, x_partial, w=None, eps=1e-6, residual_in=None, residual_out=None, out=None, mode=0):
        """sum over ranks of x_partial [N, H] (+ residual, RMSNorm when w is given) through the switch."""
        _req(x_partial, BF16, "x_partial")
        N, H = x_partial.shape
        out = torch.empty((N, H), dtype=BF16, device=x_partial.device) if out is None else out
        self._ck(self.l.nvc_nvls_allreduce_rmsnorm(self.h, _ptr(x_partial), _ptr(residual_in), _ptr(residual_out), _ptr(w),
                                                   float(eps), _ptr(out), N, H, mode, _stream()), "nvc_nvls_allreduce_rmsnorm")
        return out

    def allreduce(self, buf: torch.Tensor):
        if buf.dtype == BF16:
            self._ck(self.l.nvc_allreduce_bf16(self.h, _ptr(buf), buf.numel(), _stream()), "nvc_allreduce_bf16")
        elif buf.dtype == torch.float32:
            self._ck(self.l.nvc_allreduce_f32(self.h, _ptr(buf), buf.numel(), _stream()), "nvc_allreduce_f32")
        else:
            raise TypeError("allreduce: bf16 or f32")
        return buf

    # ---- kernels
    def embed_gather(self, ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None):
        _req(ids, torch.int32, "ids"); _req(table, BF16, "table")
        N, (V, H) = ids.numel(), table.shape
        out = torch.empty((N, H), dtype=BF16, device=table.device) if out is None else out
        self._ck(self.l.nvc_embed_gather(self.h, _ptr(ids), _ptr(table), _ptr(out), N, H, V, _stream()), "nvc_embed_gather")
        return out

    def fused_add_rmsnorm(self, x, w, eps, residual_in=None, residual_out=None, out=None):
        _req(x, BF16, "x"); _req(w, BF16, "w")
        N, H = x.shape
        out = torch.empty_like(x) if out is None else out
        self._ck(self.l.nvc_fused_add_rmsnorm(self.h, _ptr(x), _ptr(residual_in), _ptr(residual_out), _ptr(w),
                                              float(eps), _ptr(out), N, H, _stream()), "nvc_fused_add_rmsnorm")
        return out

    def gemm(self, a: torch.Tensor, w: torch.Tensor, out_dtype=BF16, out=None, force_bn=0, force_splits=0):
        """C = a @ w.T; a [M,K] (row stride allowed), w [N,K] contiguous."""
        _req(a, BF16, "a"); _req(w, BF16, "w")
        M, K = a.shape
        N = w.shape[0]
        assert w.shape[1] == K and w.is_contiguous() and a.stride(1) == 1
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        dt = 0 if out.dtype == BF16 else 1
        self._ck(self.l.nvc_gemm_bf16_ex(self.h, _ptr(a), a.stride(0), _ptr(w), _ptr(out), out.stride(0), dt,
                                         M, N, K, force_bn, force_splits, _stream()), "nvc_gemm_bf16")
        return out

    @staticmethod
    def interleave_gate_up(w_gu: torch.Tensor) -> torch.Tensor:
        """[gate; up] rows (reference layout, qwen3.rs:310) -> groups of 16 gate rows then 16 up rows,
        the layout nvc_gemm_bf16_silu_mul expects."""
        two_i, k = w_gu.shape
        i = two_i // 2
        assert i % 16 == 0
        return torch.stack([w_gu[:i].reshape(i // 16, 16, k), w_gu[i:].reshape(i // 16, 16, k)], dim=1).reshape(two_i, k).contiguous()

    def gemm_silu_mul(self, a: torch.Tensor, w_gu16: torch.Tensor, out=None, force_bn=0, force_splits=0):
        """act = silu(a @ Wgate.T) * (a @ Wup.T); w_gu16 = interleave_gate_up([gate; up])."""
        _req(a, BF16, "a"); _req(w_gu16, BF16, "w_gu16")
        M, K = a.shape
        I = w_gu16.shape[0] // 2
        assert w_gu16.shape[1] == K and w_gu16.is_contiguous() and a.stride(1) == 1
        if out is None:
            out = torch.empty((M, I), dtype=BF16, device=a.device)
        self._ck(self.l.nvc_gemm_bf16_silu_mul_ex(self.h, _ptr(a), a.stride(0), _ptr(w_gu16), _ptr(out), out.stride(0),
                                                  M, I, K, force_bn, force_splits, _stream()), "nvc_gemm_bf16_silu_mul")
        return out

    def gemm_gelu_mul(self, a: torch.Tensor, w_gu16: torch.Tensor):
        """act = gelu_tanh(a @ Wgate.T) * (a @ Wup.T); w_gu16 = interleave_gate_up([gate; up])."""
        _req(a, BF16, "a"); _req(w_gu16, BF16, "w_gu16")
        M, K = a.shape
        I = w_gu16.shape[0] // 2
        assert w_gu16.shape[1] == K and w_gu16.is_contiguous() and a.stride(1) == 1
        out = torch.empty((M, I), dtype=BF16, device=a.device)
        self._ck(self.l.nvc_gemm_bf16_gelu_mul(self.h, _ptr(a), a.stride(0), _ptr(w_gu16), _ptr(out), out.stride(0), M, I, K, _stream()),
                 "nvc_gemm_bf16_gelu_mul")
        return out

    def rope_table(self, theta: float, head_dim: int, max_pos: int, device=None):
        dev = torch.device("cuda", self.device) if device is None else device
        tab = torch.empty((max_pos, head_dim), dtype=torch.float32, device=dev)
        self._ck(self.l.nvc_rope_table_init_sync(self.h, float(theta), head_dim, max_pos, _ptr(tab)), "nvc_rope_table_init_sync")
        return tab

    def qk_norm_rope_store(self, qkv, qw, kw, eps, cos_sin, positions, nh, kv, hd,
                           slot_mapping=None, k_cache=None, v_cache=None):
        _req(qkv, BF16, "qkv"); _req(positions, torch.int32, "positions")
        N = qkv.shape[0]
        assert qkv.is_contiguous() and qkv.shape[1] == (nh + 2 * kv) * hd
        self._ck(self.l.nvc_qk_norm_rope_store(self.h, _ptr(qkv), _ptr(qw), _ptr(kw), float(eps), _ptr(cos_sin),
                                               _ptr(positions), _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache),
                                               N, nh, kv, hd, _stream()), "nvc_qk_norm_rope_store")
        return qkv

    def qkv_proj_norm_rope(self, a, w_qkv, qw, kw, eps, cos_sin, positions, nh, kv, hd, slot_mapping=None, k_cache=None,
                           v_cache=None, out=None):
        """K3 + K2: qkv = a @ w_qkv.T with q / k heads normalised + rotated and k / v scattered to the caches (one kernel at
        prefill sizes)."""
        _req(a, BF16, "a"); _req(w_qkv, BF16, "w_qkv"); _req(positions, torch.int32, "positions")
        M, K = a.shape
        N = (nh + 2 * kv) * hd
        assert w_qkv.shape == (N, K) and w_qkv.is_contiguous() and a.stride(1) == 1
        out = torch.empty((M, N), dtype=BF16, device=a.device) if out is None else out
        self._ck(self.l.nvc_qkv_proj_norm_rope(self.h, _ptr(a), a.stride(0), _ptr(w_qkv), _ptr(out), M, K, _ptr(qw), _ptr(kw),
                                               float(eps), _ptr(cos_sin), _ptr(positions), _ptr(slot_mapping), _ptr(k_cache),
                                               _ptr(v_cache), nh, kv, hd, _stream()), "nvc_qkv_proj_norm_rope")
        return out

    def store_kvcache(self, k, v, k_cache, v_cache, slot_mapping, kv, hd):
        _req(k, BF16, "k"); _req(slot_mapping, torch.int32, "slot_mapping")
        N = k.shape[0]
        assert k.stride(0) == v.stride(0)
        self._ck(self.l.nvc_store_kvcache(self.h, _ptr(k), _ptr(v), k.stride(0), _ptr(k_cache), _ptr(v_cache),
                                          _ptr(slot_mapping), N, kv, hd, _stream()), "nvc_store_kvcache")

    def prefill_attn(self, q, k, v, cu_seqlens, max_seqlen, nh, kv, hd, scale, out=None):
        """q [N, nh*hd], k/v [N, kv*hd] views (row stride allowed)."""
        _req(q, BF16, "q"); _req(cu_seqlens, torch.int32, "cu_seqlens")
        N = q.shape[0]
        B = cu_seqlens.numel() - 1
        out = torch.empty((N, nh * hd), dtype=BF16, device=q.device) if out is None else out
        self._ck(self.l.nvc_prefill_attn_varlen(self.h, _ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0),
                                                _ptr(cu_seqlens), B, N, max_seqlen, nh, kv, hd, float(scale),
                                                _ptr(out), _stream()), "nvc_prefill_attn_varlen")
        return out

    def prefill_attn_paged(self, q, k_cache, v_cache, block_tables, context_lens, cu_seqlens_q, max_seqlen_q,
                           nh, kv, hd, block_size, scale, out=None):
        """K4 over the paged cache (cached prefix): q [N, nh*hd] = the last q_len_b positions of each
        context; k_cache / v_cache [num_blocks, block_size, kv, hd] already hold the whole context."""
        _req(q, BF16, "q"); _req(cu_seqlens_q, torch.int32, "cu_seqlens_q")
        _req(block_tables, torch.int32, "block_tables"); _req(context_lens, torch.int32, "context_lens")
        N = q.shape[0]
        B = cu_seqlens_q.numel() - 1
        out = torch.empty((N, nh * hd), dtype=BF16, device=q.device) if out is None else out
        self._ck(self.l.nvc_prefill_attn_paged(self.h, _ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache),
                                               _ptr(block_tables), block_tables.shape[1], _ptr(context_lens),
                                               _ptr(cu_seqlens_q), B, N, max_seqlen_q, nh, kv, hd, block_size,
                                               k_cache.shape[0], float(scale), _ptr(out), _stream()),
                 "nvc_prefill_attn_paged")
        return out

    def prefill_attn_paged_ld(self, q, k_cache, v_cache, block_tables, context_lens, cu_seqlens_q, max_seqlen_q,
                              nh, kv, hd, block_size, scale, out):
        """The same into the left nh * hd columns of wider rows: out [N, >= nh * hd], any row stride that is a multiple of 8."""
        N, B = q.shape[0], cu_seqlens_q.numel() - 1
        self._ck(self.l.nvc_prefill_attn_paged_ld(self.h, _ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
                                                  block_tables.shape[1], _ptr(context_lens), _ptr(cu_seqlens_q), B, N, max_seqlen_q, nh,
                                                  kv, hd, block_size, k_cache.shape[0], float(scale), _ptr(out), out.stride(0), _stream()),
                 "nvc_prefill_attn_paged_ld")
        return out

    def prefill_attn_paged_sink(self, q, k_cache, v_cache, block_tables, context_lens, cu_seqlens_q, max_seqlen_q,
                                nh, kv, hd, block_size, scale, sink, out):
        """The same with one more term exp(sink_h) in every row's softmax denominator (sink: fp32 [nh] or None)."""
        N, B = q.shape[0], cu_seqlens_q.numel() - 1
        self._ck(self.l.nvc_prefill_attn_paged_sink(self.h, _ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
                                                    block_tables.shape[1], _ptr(context_lens), _ptr(cu_seqlens_q), B, N, max_seqlen_q, nh,
                                                    kv, hd, block_size, k_cache.shape[0], float(scale), _ptr(sink), _ptr(out), out.stride(0),
                                                    _stream()), "nvc_prefill_attn_paged_sink")
        return out

    def paged_decode_attn(self, q, k_cache, v_cache, block_tables, context_lens, nh, kv, hd, block_size, scale, out=None):
        _req(q, BF16, "q"); _req(block_tables, torch.int32, "block_tables"); _req(context_lens, torch.int32, "context_lens")
        B = q.shape[0]
        out = torch.empty((B, nh * hd), dtype=BF16, device=q.device) if out is None else out
        need = self.l.nvc_paged_decode_workspace_bytes(B, nh, hd, self.num_sms)
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(max(need, 1), dtype=torch.uint8, device=q.device)
        self._ck(self.l.nvc_paged_decode_attn(self.h, _ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache),
                                              _ptr(block_tables), block_tables.shape[1], _ptr(context_lens), B, nh, kv,
                                              hd, block_size, float(scale), _ptr(out), _ptr(self._ws),
                                              self._ws.numel(), _stream()), "nvc_paged_decode_attn")
        return out

    def silu_and_mul(self, x, out=None):
        _req(x, BF16, "x")
        N, I2 = x.shape
        out = torch.empty((N, I2 // 2), dtype=BF16, device=x.device) if out is None else out
        self._ck(self.l.nvc_silu_and_mul(self.h, _ptr(x), _ptr(out), N, I2 // 2, _stream()), "nvc_silu_and_mul")
        return out

    def gather_rows(self, x, residual, rows):
        _req(x, BF16, "x"); _req(rows, torch.int32, "rows")
        B, H = rows.numel(), x.shape[1]
        xo = torch.empty((B, H), dtype=BF16, device=x.device)
        ro = None if residual is None else torch.empty((B, H), dtype=torch.float32, device=x.device)
        self._ck(self.l.nvc_gather_rows(self.h, _ptr(x), _ptr(residual), _ptr(rows), _ptr(xo), _ptr(ro), B, H, _stream()),
                 "nvc_gather_rows")
        return xo, ro

    def argmax_last(self, logits, index_offset=0):
        _req(logits, torch.float32, "logits")
        B, V = logits.shape
        idx = torch.empty((B,), dtype=torch.int32, device=logits.device)
        val = torch.empty((B,), dtype=torch.float32, device=logits.device)
        self._ck(self.l.nvc_argmax_last(self.h, _ptr(logits), logits.stride(0), _ptr(idx), _ptr(val), B, V,
                                        index_offset, _stream()), "nvc_argmax_last")
        return idx, val

    def sample_gumbel(self, logits, temperatures, streams, seed: int, index_offset=0):
        """K8s: seeded Gumbel-max draw per row; streams: int64 tensor holding the u64 stream ids."""
        _req(logits, torch.float32, "logits"); _req(temperatures, torch.float32, "temperatures")
        _req(streams, torch.int64, "streams")
        B, V = logits.shape
        idx = torch.empty((B,), dtype=torch.int32, device=logits.device)
        val = torch.empty((B,), dtype=torch.float32, device=logits.device)
        self._ck(self.l.nvc_sample_gumbel(self.h, _ptr(logits), logits.stride(0), _ptr(temperatures), _ptr(streams),
                                          C.c_uint64(seed & (2 ** 64 - 1)), _ptr(idx), _ptr(val), B, V, index_offset,
                                          _stream()), "nvc_sample_gumbel")
        return idx, val


# ----------------------------------------------------------------------------- fp32-residual mechanisms
# (Dynamic-Tanh norm, latent attention, mixture-of-experts routing, the FMA matrix products of the exact mode).
# Tensors are torch.bfloat16 (serving) or torch.float32 (exact mode); the dtype of the data picks the kernel.
ACT_NONE, ACT_RELU2, ACT_GELU_TANH_MUL = 0, 1, 2


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return 0
    if t.dtype == torch.float32:
        return 1
    raise TypeError(f"bf16 or fp32 expected, got {t.dtype}")


def embed_gather_f32(ctx, ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    N, H = ids.numel(), table.shape[1]
    out = torch.empty(N, H, dtype=torch.float32, device=table.device)
    check(ctx.l.nvc_embed_gather_f32(ctx.h, _ptr(ids), _ptr(table), _dt(table), table.stride(0), _ptr(out), H, N, H, _stream()),
          "nvc_embed_gather_f32", ctx.h)
    return out


def dyt_norm(ctx, res: torch.Tensor, addends, w, b, alpha, out_dtype=torch.bfloat16, rows=None, write_back=True):
    """(updated residual or None, normed rows or None): residual += sum(addends); DyT of the rows when w is given."""
    N = res.shape[0] if rows is None else rows.numel()
    H = res.shape[1]
    a = list(addends) + [None] * (3 - len(addends))
    out = torch.empty(N, H, dtype=out_dtype, device=res.device) if w is not None else None
    ro = res if (write_back and rows is None) else None
    check(ctx.l.nvc_dyt_norm(ctx.h, _ptr(res), _ptr(a[0]), _ptr(a[1]), _ptr(a[2]), _ptr(ro), res.stride(0), _ptr(w), _ptr(b),
                             _ptr(alpha), _ptr(out), _dt(out) if out is not None else 0, H, _ptr(rows), N, H, _stream()),
          "nvc_dyt_norm", ctx.h)
    return ro, out


def latent_norm_store(ctx, x: torch.Tensor, n0: int, off1: int, n1: int, w0, w1, eps: float, cache, slot_mapping, dtype):
    """x: fp32 [N, ld]; returns the normed query latent [N, n0]; the key/value latent goes to cache[slot]."""
    N = x.shape[0]
    out0 = torch.empty(N, n0, dtype=dtype, device=x.device)
    check(ctx.l.nvc_latent_norm_store(ctx.h, _ptr(x), x.stride(0), n0, off1, n1, _ptr(w0), _ptr(w1), eps, _ptr(out0), n0,
                                      _ptr(cache), cache.stride(0) if cache is not None else 0, _ptr(slot_mapping), _dt(out0), N,
                                      _stream()), "nvc_latent_norm_store", ctx.h)
    return out0


def act_mul(ctx, x: torch.Tensor, F: int, kind: int) -> torch.Tensor:
    N = x.shape[0]
    out = torch.empty(N, F, dtype=x.dtype, device=x.device)
    check(ctx.l.nvc_act_mul(ctx.h, _ptr(x), x.stride(0), _ptr(out), F, _dt(x), N, F, F, kind, _stream()), "nvc_act_mul", ctx.h)
    return out


def linear(ctx, A: torch.Tensor, W: torch.Tensor, out_dtype=None, act: int = ACT_NONE) -> torch.Tensor:
    """A [M, K] or [batch, M, K]; W [N, K] or [batch, N, K]: act(A . W^T) on the FMA pipe."""
    batched = A.dim() == 3
    Bn = A.shape[0] if batched else 1
    M, K, N = A.shape[-2], A.shape[-1], W.shape[-2]
    out_dtype = out_dtype or A.dtype
    C_ = torch.empty((Bn, M, N) if batched else (M, N), dtype=out_dtype, device=A.device)
    check(ctx.l.nvc_linear(ctx.h, _ptr(A), A.stride(-2), A.stride(0) if batched else 0, _ptr(W), W.stride(-2),
                           W.stride(0) if batched else 0, _ptr(C_), N, M * N if batched else 0, _dt(A), _dt(C_), M, N, K, Bn, act,
                           _stream()), "nvc_linear", ctx.h)
    return C_


def linear_grouped(ctx, A, a_rows, W, offsets, rows: int, out_dtype=None, act: int = ACT_NONE) -> torch.Tensor:
    """W [groups, N, K]; rows [offsets[g], offsets[g + 1]) of the result use W[g] on A[a_rows[r]]."""
    G, N, K = W.shape
    out_dtype = out_dtype or A.dtype
    C_ = torch.zeros(rows, N, dtype=out_dtype, device=A.device)
    check(ctx.l.nvc_linear_grouped(ctx.h, _ptr(A), A.stride(0), _ptr(a_rows), _ptr(W), K, N * K, _ptr(C_), N, _ptr(offsets), G, rows,
                                   _dt(A), _dt(C_), N, K, act, _stream()), "nvc_linear_grouped", ctx.h)
    return C_


def moe_route(ctx, h, w_router, correction, w_gate, top: int, scale: float):
    N, H = h.shape
    E = w_router.shape[0]
    idx = torch.empty(N, top, dtype=torch.int32, device=h.device)
    w = torch.empty(N, top, dtype=torch.float32, device=h.device)
    gate = torch.empty(N, dtype=torch.float32, device=h.device) if w_gate is not None else None
    check(ctx.l.nvc_moe_route(ctx.h, _ptr(h), _dt(h), h.stride(0), _ptr(w_router), _ptr(correction), _ptr(w_gate), E, top, scale,
                              _ptr(idx), _ptr(w), _ptr(gate), N, H, _stream()), "nvc_moe_route", ctx.h)
    return idx, w, gate


def moe_route_logits(ctx, z: torch.Tensor, correction, E: int, top: int, scale: float, gate_col: int = -1):
    """z: fp32 [N, >= E] router logits (column gate_col: the shared gate's logit)."""
    N = z.shape[0]
    idx = torch.empty(N, top, dtype=torch.int32, device=z.device)
    w = torch.empty(N, top, dtype=torch.float32, device=z.device)
    gate = torch.empty(N, dtype=torch.float32, device=z.device) if gate_col >= 0 else None
    check(ctx.l.nvc_moe_route_logits(ctx.h, _ptr(z), z.stride(0), _ptr(correction), E, top, scale, gate_col, _ptr(idx), _ptr(w), _ptr(gate),
                                     N, _stream()), "nvc_moe_route_logits", ctx.h)
    return idx, w, gate


def moe_sort(ctx, idx: torch.Tensor, E: int):
    N, top = idx.shape
    offsets = torch.empty(E + 1, dtype=torch.int32, device=idx.device)
    src = torch.empty(N * top, dtype=torch.int32, device=idx.device)
    pos = torch.empty(N * top, dtype=torch.int32, device=idx.device)
    check(ctx.l.nvc_moe_sort(ctx.h, _ptr(idx), N, top, E, _ptr(offsets), _ptr(src), _ptr(pos), _stream()), "nvc_moe_sort", ctx.h)
    return offsets, src, pos


def moe_sort_padded(ctx, idx: torch.Tensor, E: int, align: int = 128):
    """Groups padded to multiples of `align` rows: (offsets [E + 1], src [tiles * align] with -1 in the padding, pos, tile_group)."""
    N, top = idx.shape
    tiles = (N * top + E * (align - 1) + align - 1) // align
    offsets = torch.empty(E + 1, dtype=torch.int32, device=idx.device)
    src = torch.full((tiles * align,), -7, dtype=torch.int32, device=idx.device)
    pos = torch.empty(N * top, dtype=torch.int32, device=idx.device)
    tile_group = torch.full((tiles,), -7, dtype=torch.int32, device=idx.device)
    check(ctx.l.nvc_moe_sort_padded(ctx.h, _ptr(idx), N, top, E, align, _ptr(offsets), _ptr(src), _ptr(pos), _ptr(tile_group), tiles,
                                    _stream()), "nvc_moe_sort_padded", ctx.h)
    return offsets, src, pos, tile_group


def gather_rows(ctx, x: torch.Tensor, src: torch.Tensor, num_rows: torch.Tensor) -> torch.Tensor:
    """out[r] = x[src[r]] for r < num_rows[0] (zeros where src[r] < 0); rows behind num_rows keep the fill value."""
    out = torch.full((src.numel(), x.shape[1]), 3.0, dtype=x.dtype, device=x.device)
    check(ctx.l.nvc_gather_rows_bf16(ctx.h, _ptr(x), x.stride(0), _ptr(src), _ptr(num_rows), _ptr(out), out.stride(0), src.numel(),
                                     x.shape[1], _stream()), "nvc_gather_rows_bf16", ctx.h)
    return out


def gemm_act(ctx, A, W, act: int = ACT_NONE, out_dtype=None) -> torch.Tensor:
    """act(A W^T) on the tcgen05 kernels, the activation in the epilogue."""
    M, K = A.shape
    N = W.shape[0]
    C_ = torch.empty(M, N, dtype=out_dtype or A.dtype, device=A.device)
    check(ctx.l.nvc_gemm_bf16_act(ctx.h, _ptr(A), A.stride(0), _ptr(W), _ptr(C_), N, _dt(C_), M, N, K, act, _stream()),
          "nvc_gemm_bf16_act", ctx.h)
    return C_


def gemm_grouped(ctx, A, W, tile_group, act: int = ACT_NONE, out_dtype=None) -> torch.Tensor:
    """A [tiles * 128, K] sorted by group (groups padded to 128 rows), W [groups, N, K]: act(A[r] . W[tile_group[r // 128]]^T)."""
    G, N, K = W.shape
    C_ = torch.zeros(A.shape[0], N, dtype=out_dtype or A.dtype, device=A.device)
    check(ctx.l.nvc_gemm_bf16_grouped(ctx.h, _ptr(A), A.stride(0), _ptr(W), _ptr(C_), N, _dt(C_), A.shape[0], N, K, _ptr(tile_group), G, act,
                                      _stream()), "nvc_gemm_bf16_grouped", ctx.h)
    return C_


def moe_combine(ctx, y, pos, w, shared=None, gate=None) -> torch.Tensor:
    N, top = w.shape
    H = y.shape[1]
    out = torch.empty(N, H, dtype=torch.float32, device=y.device)
    check(ctx.l.nvc_moe_combine(ctx.h, _ptr(y), _dt(y), y.stride(0), _ptr(pos), _ptr(w), top, _ptr(shared),
                                _dt(shared) if shared is not None else 0, shared.stride(0) if shared is not None else 0, _ptr(gate),
                                _ptr(out), H, N, H, _stream()), "nvc_moe_combine", ctx.h)
    return out


def latent_attn_paged(ctx, q, cache, block_tables, context_lens, cu_seqlens, max_qlen: int, block_size: int, scale: float,
                      workspace: Optional[torch.Tensor] = None):
    """q: [rows, heads, D]; cache: [slots, >= D]; returns the attended latents [rows, heads, D]."""
    rows, heads, D = q.shape
    out = torch.empty_like(q)
    B = context_lens.numel()
    check(ctx.l.nvc_latent_attn_paged(ctx.h, _ptr(q), heads * D, _ptr(cache), cache.stride(0), _ptr(block_tables),
                                      block_tables.stride(0), _ptr(context_lens), _ptr(cu_seqlens), B, max_qlen, heads, D, D,
                                      block_size, scale, _ptr(out), heads * D, _dt(q), _ptr(workspace),
                                      workspace.numel() * workspace.element_size() if workspace is not None else 0, _stream()),
          "nvc_latent_attn_paged", ctx.h)
    return out


# ---------------------------------------------------------------- RMS-norm pair, q / k / v preparation, wide attention, retention
class QkvPrepC(C.Structure):
    """nvc_qkv_prep of include/nvc_b200.h."""
    _fields_ = [("in_", C.c_void_p), ("ldi", C.c_int), ("bias", C.c_void_p), ("q_off", C.c_int), ("k_off", C.c_int), ("v_off", C.c_int),
                ("q_heads", C.c_int), ("kv_heads", C.c_int), ("dim", C.c_int), ("vdim", C.c_int), ("q_norm", C.c_void_p),
                ("k_norm", C.c_void_p), ("eps", C.c_float), ("rot_dims", C.c_int), ("rot_half", C.c_int), ("rot_table", C.c_void_p),
                ("positions", C.c_void_p), ("k_scale", C.c_float), ("blend", C.c_int), ("lambda_", C.c_void_p), ("v_first", C.c_void_p),
                ("ldvf", C.c_int), ("q_out", C.c_void_p), ("ldq", C.c_int), ("k_out", C.c_void_p), ("v_out", C.c_void_p), ("ldk", C.c_int),
                ("ldv", C.c_int), ("slot_mapping", C.c_void_p), ("q_dtype", C.c_int), ("kv_dtype", C.c_int), ("v_scale", C.c_float),
                ("unit_norm", C.c_int), ("act", C.c_int)]


class AttnSpecC(C.Structure):
    """nvc_attn_spec of include/nvc_b200.h."""
    _fields_ = [("heads", C.c_int), ("kv_heads", C.c_int), ("dim", C.c_int), ("vdim", C.c_int), ("scale", C.c_float), ("window", C.c_int),
                ("sink", C.c_void_p), ("gate", C.c_void_p), ("ldg", C.c_int), ("out_scale", C.c_float), ("softcap", C.c_float),
                ("chunk", C.c_int), ("gate_per_head", C.c_int)]


def _a(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def embed_gather_scaled_f32(ctx, ids, table, scale: float):
    out = torch.empty(ids.numel(), table.shape[1], dtype=torch.float32, device=table.device)
    check(ctx.l.nvc_embed_gather_scaled_f32(ctx.h, _ptr(ids), _ptr(table), _dt(table), table.stride(0), scale, _ptr(out), out.stride(0),
                                            ids.numel(), table.shape[1], _stream()), "nvc_embed_gather_scaled_f32", ctx.h)
    return out


def rms_norm_pair(ctx, res, addends, w0, w1=None, eps: float = 1e-5, out_dtype=torch.float32, rows=None, write_back: bool = True):
    """(residual after the sums - a new tensor, or None when rows gather or write_back is False; out0; out1)."""
    a0, a1 = (list(addends) + [None, None])[:2]
    N = res.shape[0] if rows is None else rows.numel()
    H = res.shape[1]
    res_out = torch.empty_like(res) if (rows is None and write_back) else None
    out0 = torch.empty(N, H, dtype=out_dtype, device=res.device) if w0 is not None else None
    out1 = torch.empty(N, H, dtype=out_dtype, device=res.device) if w1 is not None else None
    check(ctx.l.nvc_rms_norm_pair(ctx.h, _ptr(res), _ptr(a0), _ptr(a1), _ptr(res_out), res.stride(0), _ptr(w0), _ptr(out0), _ptr(w1),
                                  _ptr(out1), 0 if out_dtype == torch.bfloat16 else 1, H, eps, _ptr(rows), N, H, _stream()),
          "nvc_rms_norm_pair", ctx.h)
    return res_out, out0, out1


def head_gate(ctx, o, gate, heads: int, vdim: int, norm: bool, eps: float, act: str, out_scale: float, out_dtype=torch.float32):
    out = torch.empty(o.shape[0], heads * vdim, dtype=out_dtype, device=o.device)
    check(ctx.l.nvc_head_gate(ctx.h, _ptr(o), o.stride(0), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(out), out.stride(0),
                              0 if out_dtype == torch.bfloat16 else 1, heads, vdim, 1 if norm else 0, eps, {"sigmoid": 0, "silu": 1}[act],
                              out_scale, o.shape[0], _stream()), "nvc_head_gate", ctx.h)
    return out


def rotary_table(ctx, base: float, dims: int, max_pos: int, device="cuda:0"):
    out = torch.empty(max_pos, dims // 2, 2, dtype=torch.float32, device=device)
    check(ctx.l.nvc_rotary_table_init_sync(ctx.h, base, dims, max_pos, _ptr(out)), "nvc_rotary_table_init_sync", ctx.h)
    return out


def qkv_prep(ctx, x, q_off, k_off, v_off, q_heads, kv_heads, dim, vdim, q_out, k_out, v_out, *, bias=None, q_norm=None, k_norm=None,
             eps=1e-5, rot_dims=0, rot_half=False, rot_table=None, positions=None, k_scale=1.0, blend=0, lam=None, v_first=None,
             slot_mapping=None, v_scale=1.0, unit_norm=False, silu=False):
    """x: fp32 [N, ld] rows of a fused projection; q_out [N, q_heads * dim]; k_out / v_out: cache rows (slot_mapping) or [N, ...]."""
    p = QkvPrepC(_a(x), x.stride(0), _a(bias), q_off, k_off, v_off, q_heads, kv_heads, dim, vdim, _a(q_norm), _a(k_norm), eps, rot_dims,
                 1 if rot_half else 0, _a(rot_table), _a(positions), k_scale, blend, _a(lam), _a(v_first),
                 v_first.stride(0) if v_first is not None else 0, _a(q_out), q_out.stride(0), _a(k_out), _a(v_out), k_out.stride(0),
                 v_out.stride(0), _a(slot_mapping), _dt(q_out), _dt(k_out), v_scale, 1 if unit_norm else 0, 1 if silu else 0)
    check(ctx.l.nvc_qkv_prep_run(ctx.h, C.byref(p), x.shape[0], _stream()), "nvc_qkv_prep_run", ctx.h)


def attn_paged_wide(ctx, q, k_cache, v_cache, block_tables, context_lens, cu_seqlens, max_qlen: int, block_size: int, heads: int,
                    kv_heads: int, dim: int, vdim: int, scale: float, window: int = 0, sink=None, gate=None, out_scale: float = 1.0,
                    softcap: float = 0.0, chunk: int = 0, gate_per_head: bool = False):
    """q: [rows, heads * dim]; k_cache [slots, kv_heads * dim], v_cache [slots, kv_heads * vdim]; returns [rows, heads * vdim]."""
    rows = q.shape[0]
    out = torch.empty(rows, heads * vdim, dtype=q.dtype, device=q.device)
    sp = AttnSpecC(heads, kv_heads, dim, vdim, scale, window, _a(sink), _a(gate), gate.stride(0) if gate is not None else 0, out_scale,
                   softcap, chunk, 1 if gate_per_head else 0)
    check(ctx.l.nvc_attn_paged_wide(ctx.h, _ptr(q), q.stride(0), _ptr(k_cache), k_cache.stride(0), _ptr(v_cache), v_cache.stride(0),
                                    _ptr(block_tables), block_tables.stride(0), _ptr(context_lens), _ptr(cu_seqlens), context_lens.numel(),
                                    rows, max_qlen, block_size, C.byref(sp), _ptr(out), out.stride(0), _dt(q), _stream()),
          "nvc_attn_paged_wide", ctx.h)
    return out


def retention_scan(ctx, q, k, v, state, state_slots, cu_seqlens, positions, decay, heads: int, dim: int, vdim: int, max_qlen: int = 1 << 20):
    """q, k: fp32 [N, heads * dim]; v: fp32 [N, heads * vdim]; state: fp32 [slots, heads, dim, vdim], updated in place."""
    o = torch.empty(q.shape[0], heads * vdim, dtype=torch.float32, device=q.device)
    check(ctx.l.nvc_retention_scan(ctx.h, _ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(o), o.stride(0), _ptr(state),
                                   _ptr(state_slots), _ptr(cu_seqlens), _ptr(positions), _ptr(decay), state_slots.numel(), max_qlen, heads, dim, vdim,
                                   _stream()), "nvc_retention_scan", ctx.h)
    return o


# ---------------------------------------------------------------- sandwich norms, rotary latent rows, delta rule, softmax routing
ACT_GELU_TANH, ACT_GLU_CLAMP = 3, 4
ROUTE_SIGMOID, ROUTE_SOFTMAX = 0, 1


class DeltaPrepC(C.Structure):
    """nvc_delta_prep of include/nvc_b200.h."""
    _fields_ = [("in_", C.c_void_p), ("ldi", C.c_int), ("q_off", C.c_int), ("k_off", C.c_int), ("v_off", C.c_int), ("b_off", C.c_int),
                ("a_off", C.c_int), ("heads", C.c_int), ("kv_heads", C.c_int), ("dim", C.c_int), ("vdim", C.c_int), ("taps", C.c_int),
                ("conv_w", C.c_void_p), ("conv_state", C.c_void_p), ("state_slots", C.c_void_p), ("cu_seqlens", C.c_void_p),
                ("positions", C.c_void_p), ("A_log", C.c_void_p), ("dt_bias", C.c_void_p), ("unit_eps", C.c_float), ("q_scale", C.c_float),
                ("q_out", C.c_void_p), ("k_out", C.c_void_p), ("v_out", C.c_void_p), ("ldq", C.c_int), ("ldk", C.c_int), ("ldv", C.c_int),
                ("gb_out", C.c_void_p), ("B", C.c_int)]


def rms_norm_sandwich(ctx, res, y, wy, w, eps: float = 1e-5, weight_offset: float = 1.0, out_dtype=torch.float32, rows=None,
                      write_back: bool = True):
    """(residual after the sum - a new tensor, or None when rows gather or write_back is False; the normed rows or None)."""
    N = res.shape[0] if rows is None else rows.numel()
    H = res.shape[1]
    res_out = torch.empty_like(res) if (rows is None and write_back) else None
    out = torch.empty(N, H, dtype=out_dtype, device=res.device) if w is not None else None
    check(ctx.l.nvc_rms_norm_sandwich(ctx.h, _ptr(res), _ptr(y), _ptr(wy), _ptr(res_out), res.stride(0), _ptr(w), _ptr(out),
                                      0 if out_dtype == torch.bfloat16 else 1, H, eps, weight_offset, _ptr(rows), N, H, _stream()),
          "nvc_rms_norm_sandwich", ctx.h)
    return res_out, out


def latent_norm_store_rot(ctx, x, n0: int, off1: int, n1: int, w0, w1, eps: float, cache, slot_mapping, rot_dim: int, rot_dims: int,
                          rot_half: bool, rot_table, positions, dtype):
    """x: fp32 [N, ld]; returns the normed query latent [N, n0]; [normed latent | rotated part] goes to cache[slot]."""
    N = x.shape[0]
    out0 = torch.empty(N, n0, dtype=dtype, device=x.device)
    check(ctx.l.nvc_latent_norm_store_rot(ctx.h, _ptr(x), x.stride(0), n0, off1, n1, _ptr(w0), _ptr(w1), eps, _ptr(out0), n0, _ptr(cache),
                                          cache.stride(0) if cache is not None else 0, _ptr(slot_mapping), rot_dim, rot_dims,
                                          1 if rot_half else 0, _ptr(rot_table), _ptr(positions), _dt(out0), N, _stream()),
          "nvc_latent_norm_store_rot", ctx.h)
    return out0


def head_split_rot(ctx, x, heads: int, dim: int, rot_dim: int, rot_dims: int, rot_half: bool, rot_table, positions, out_a, hs_a: int, out_b,
                   hs_b: int, off_b: int):
    check(ctx.l.nvc_head_split_rot(ctx.h, _ptr(x), x.stride(0), heads, dim, rot_dim, rot_dims, 1 if rot_half else 0, _ptr(rot_table),
                                   _ptr(positions), _ptr(out_a), out_a.stride(0), hs_a, _ptr(out_b), out_b.stride(0), hs_b, off_b, _dt(out_a),
                                   x.shape[0], _stream()), "nvc_head_split_rot", ctx.h)


def head_gate_w(ctx, o, gate, weight, heads: int, vdim: int, norm: bool, eps: float, act: str, out_scale: float, out_dtype=torch.float32):
    out = torch.empty(o.shape[0], heads * vdim, dtype=out_dtype, device=o.device)
    check(ctx.l.nvc_head_gate_w(ctx.h, _ptr(o), o.stride(0), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(weight), _ptr(out),
                                out.stride(0), 0 if out_dtype == torch.bfloat16 else 1, heads, vdim, 1 if norm else 0, eps,
                                {"sigmoid": 0, "silu": 1}[act], out_scale, o.shape[0], _stream()), "nvc_head_gate_w", ctx.h)
    return out


def act_mul_p(ctx, x, F: int, Fp: int, kind: int, p0: float = 0.0, p1: float = 0.0):
    N = x.shape[0]
    out = torch.empty(N, F, dtype=x.dtype, device=x.device)
    check(ctx.l.nvc_act_mul_p(ctx.h, _ptr(x), x.stride(0), _ptr(out), F, _dt(x), N, F, Fp, kind, p0, p1, _stream()), "nvc_act_mul_p", ctx.h)
    return out


def moe_route_logits_ex(ctx, z, correction, E: int, top: int, scale: float, score: int, normalize: bool):
    N = z.shape[0]
    idx = torch.empty(N, top, dtype=torch.int32, device=z.device)
    w = torch.empty(N, top, dtype=torch.float32, device=z.device)
    check(ctx.l.nvc_moe_route_logits_ex(ctx.h, _ptr(z), z.stride(0), _ptr(correction), E, top, scale, -1, score, 1 if normalize else 0, _ptr(idx),
                                        _ptr(w), None, N, _stream()), "nvc_moe_route_logits_ex", ctx.h)
    return idx, w


def moe_sort_padded_ex(ctx, idx, E: int, E_real: int, align: int = 128):
    N, top = idx.shape
    tiles = (N * top + E * (align - 1) + align - 1) // align
    offsets = torch.empty(E + 1, dtype=torch.int32, device=idx.device)
    src = torch.full((tiles * align,), -7, dtype=torch.int32, device=idx.device)
    pos = torch.empty(N * top, dtype=torch.int32, device=idx.device)
    tile_group = torch.full((tiles,), -7, dtype=torch.int32, device=idx.device)
    check(ctx.l.nvc_moe_sort_padded_ex(ctx.h, _ptr(idx), N, top, E, E_real, align, _ptr(offsets), _ptr(src), _ptr(pos), _ptr(tile_group), tiles,
                                       _stream()), "nvc_moe_sort_padded_ex", ctx.h)
    return offsets, src, pos, tile_group


def moe_combine_identity(ctx, y, pos, w, idx, E_real: int, x):
    N, top = w.shape
    H = x.shape[1]
    out = torch.empty(N, H, dtype=torch.float32, device=y.device)
    check(ctx.l.nvc_moe_combine_identity(ctx.h, _ptr(y), _dt(y), y.stride(0), _ptr(pos), _ptr(w), _ptr(idx), top, E_real, _ptr(x), _dt(x),
                                         x.stride(0), _ptr(out), H, N, H, _stream()), "nvc_moe_combine_identity", ctx.h)
    return out


def delta_rule(ctx, x, offs, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, conv_w, conv_state, state, state_slots, cu_seqlens,
               positions, A_log, dt_bias, unit_eps: float = 1e-6, q_scale: Optional[float] = None, max_qlen: int = 1 << 20):
    """x: fp32 [N, ld] rows of the fused projection, offs = (q, k, v, beta, a) columns; conv_w: [taps, C] (tap-major).  Runs the
    preparation and the recurrence;
    conv_state [slots, taps - 1, C] and state [slots, heads, dim, vdim] are updated in place.  Returns (o [N, heads * vdim], q, k, v, gb)."""
    N = x.shape[0]
    dev = x.device
    q = torch.empty(N, kv_heads * dim, dtype=torch.float32, device=dev)
    k = torch.empty_like(q)
    v = torch.empty(N, heads * vdim, dtype=torch.float32, device=dev)
    gb = torch.empty(N, 2 * heads, dtype=torch.float32, device=dev)
    o = torch.empty(N, heads * vdim, dtype=torch.float32, device=dev)
    p = DeltaPrepC(_a(x), x.stride(0), offs[0], offs[1], offs[2], offs[3], offs[4], heads, kv_heads, dim, vdim, taps, _a(conv_w), _a(conv_state),
                   _a(state_slots), _a(cu_seqlens), _a(positions), _a(A_log), _a(dt_bias), unit_eps, dim ** -0.5 if q_scale is None else q_scale,
                   _a(q), _a(k), _a(v), q.stride(0), k.stride(0), v.stride(0), _a(gb), state_slots.numel())
    longest = int((cu_seqlens[1:] - cu_seqlens[:-1]).max().item()) if cu_seqlens is not None else 1
    check(ctx.l.nvc_delta_prep_run(ctx.h, C.byref(p), N, longest, _stream()), "nvc_delta_prep_run", ctx.h)
    check(ctx.l.nvc_delta_rule_scan(ctx.h, C.byref(p), _ptr(o), o.stride(0), _ptr(state), max_qlen, _stream()), "nvc_delta_rule_scan", ctx.h)
    return o, q, k, v, gb


# ---------------------------------------------------------------- blended norms, grouped gated norms, decayed scans, state space preparation
ACT_SILU_MUL = 5


class DecayScanC(C.Structure):
    """nvc_decay_scan_args of include/nvc_b200.h."""
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("ldq", C.c_int), ("ldk", C.c_int), ("ldv", C.c_int), ("o", C.c_void_p),
                ("ldo", C.c_int), ("state", C.c_void_p), ("state_slots", C.c_void_p), ("cu_seqlens", C.c_void_p), ("positions", C.c_void_p),
                ("decay", C.c_void_p), ("log_decay", C.c_void_p), ("ldl", C.c_int), ("skip", C.c_void_p), ("skip_w", C.c_void_p), ("lds", C.c_int),
                ("heads", C.c_int), ("qk_heads", C.c_int), ("dim", C.c_int), ("vdim", C.c_int)]


class SsdPrepC(C.Structure):
    """nvc_ssd_prep of include/nvc_b200.h."""
    _fields_ = [("in_", C.c_void_p), ("ldi", C.c_int), ("xbc_off", C.c_int), ("dt_off", C.c_int), ("heads", C.c_int), ("vdim", C.c_int),
                ("groups", C.c_int), ("state", C.c_int), ("taps", C.c_int), ("conv_w", C.c_void_p), ("conv_b", C.c_void_p),
                ("conv_state", C.c_void_p), ("state_slots", C.c_void_p), ("cu_seqlens", C.c_void_p), ("positions", C.c_void_p),
                ("A_log", C.c_void_p), ("dt_bias", C.c_void_p), ("x_out", C.c_void_p), ("v_out", C.c_void_p), ("ldx", C.c_int),
                ("b_out", C.c_void_p), ("c_out", C.c_void_p), ("ldbc", C.c_int), ("log_decay", C.c_void_p), ("ldl", C.c_int), ("B", C.c_int)]


def rms_norm_blend(ctx, res, y0=None, w0=None, c0: float = 1.0, y1=None, w1=None, c1: float = 1.0, w=None, bias=None, eps: float = 1e-5,
                   out_dtype=torch.float32, rows=None, write_back: bool = True, plain_out: bool = False):
    """(residual after the sums - a new tensor, or None when rows gather or write_back is False; the normed rows - or the sum itself in
    out_dtype when plain_out - or None)."""
    ref = res if res is not None else y0
    N = ref.shape[0] if rows is None else rows.numel()
    H = ref.shape[1]
    res_out = torch.empty_like(ref) if (rows is None and write_back) else None
    out = torch.empty(N, H, dtype=out_dtype, device=ref.device) if (w is not None or plain_out) else None
    check(ctx.l.nvc_rms_norm_blend(ctx.h, _ptr(res), _ptr(bias), _ptr(y0), _ptr(w0), c0, _ptr(y1), _ptr(w1), c1, _ptr(res_out), ref.stride(0),
                                   _ptr(w), _ptr(out), 0 if out_dtype == torch.bfloat16 else 1, H, eps, _ptr(rows), N, H, _stream()),
          "nvc_rms_norm_blend", ctx.h)
    return res_out, out


def group_norm_gate(ctx, o, gate, weight, groups: int, gsize: int, gate_first: bool, eps: float, act: str, out_dtype=torch.float32):
    out = torch.empty(o.shape[0], groups * gsize, dtype=out_dtype, device=o.device)
    check(ctx.l.nvc_group_norm_gate(ctx.h, _ptr(o), o.stride(0), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(weight), _ptr(out),
                                    out.stride(0), 0 if out_dtype == torch.bfloat16 else 1, groups, gsize, 1 if gate_first else 0, eps,
                                    {"sigmoid": 0, "silu": 1}[act], o.shape[0], _stream()), "nvc_group_norm_gate", ctx.h)
    return out


def decay_scan(ctx, q, k, v, state, state_slots, cu_seqlens, positions, heads: int, qk_heads: int, dim: int, vdim: int, decay=None,
               log_decay=None, skip=None, skip_w=None, max_qlen: int = 1 << 20):
    """q, k: fp32 [N, qk_heads * dim]; v: fp32 [N, heads * vdim]; decay [heads] or log_decay [N, heads]; state updated in place."""
    o = torch.empty(q.shape[0], heads * vdim, dtype=torch.float32, device=q.device)
    p = DecayScanC(_a(q), _a(k), _a(v), q.stride(0), k.stride(0), v.stride(0), _a(o), o.stride(0), _a(state), _a(state_slots), _a(cu_seqlens),
                   _a(positions), _a(decay), _a(log_decay), log_decay.stride(0) if log_decay is not None else 0, _a(skip), _a(skip_w),
                   skip.stride(0) if skip is not None else 0, heads, qk_heads, dim, vdim)
    check(ctx.l.nvc_decay_scan(ctx.h, C.byref(p), state_slots.numel(), max_qlen, _stream()), "nvc_decay_scan", ctx.h)
    return o


def ssd_prep(ctx, x, xbc_off: int, dt_off: int, heads: int, vdim: int, groups: int, state: int, taps: int, conv_w, conv_b, conv_state,
             state_slots, cu_seqlens, positions, A_log, dt_bias):
    """x: fp32 [N, ld] rows of the fused projection; conv_w [taps, C] tap-major; conv_state [slots, taps - 1, C] is advanced in place.
    Returns (x, v = dt x, B, C, log_decay)."""
    N, dev = x.shape[0], x.device
    inner, gn = heads * vdim, groups * state
    xo = torch.empty(N, inner, dtype=torch.float32, device=dev)
    vo = torch.empty_like(xo)
    bo = torch.empty(N, gn, dtype=torch.float32, device=dev)
    co = torch.empty_like(bo)
    ld = torch.empty(N, heads, dtype=torch.float32, device=dev)
    p = SsdPrepC(_a(x), x.stride(0), xbc_off, dt_off, heads, vdim, groups, state, taps, _a(conv_w), _a(conv_b), _a(conv_state), _a(state_slots),
                 _a(cu_seqlens), _a(positions), _a(A_log), _a(dt_bias), _a(xo), _a(vo), inner, _a(bo), _a(co), gn, _a(ld), heads,
                 state_slots.numel())
    check(ctx.l.nvc_ssd_prep_run(ctx.h, C.byref(p), N, _stream()), "nvc_ssd_prep_run", ctx.h)
    check(ctx.l.nvc_ssd_conv_advance(ctx.h, C.byref(p), _stream()), "nvc_ssd_conv_advance", ctx.h)
    return xo, vo, bo, co, ld


def moe_scatter_scaled(ctx, h, pos, w, rows: int):
    """out[pos[n * top + t]] = w[n, t] * h[n]; `rows` rows of output (zeros elsewhere)."""
    N, top = w.shape
    out = torch.zeros(rows, h.shape[1], dtype=h.dtype, device=h.device)
    check(ctx.l.nvc_moe_scatter_scaled(ctx.h, _ptr(h), _dt(h), h.stride(0), _ptr(pos), _ptr(w), top, _ptr(out), out.stride(0), N, h.shape[1],
                                       _stream()), "nvc_moe_scatter_scaled", ctx.h)
    return out
