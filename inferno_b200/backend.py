"""Host-side mirror of the reference's backend operator surface for the attention path.

`CudaBackend` plays the role of the reference's `MetalBackend` (crates/backend/src/backend.rs:2175)
for the methods of `trait Backend` that lie on the attention path; method names follow the trait.
Every method is a thin shim over one C-ABI call of libinferno_attn.so.  torch is used for device
memory and stream plumbing only: tensors are handed to the library as raw device pointers.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import lib as L
from .lib import InfernoError


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return None
    assert t.is_cuda and t.is_contiguous(), "device tensors must be contiguous CUDA tensors"
    return C.c_void_p(t.data_ptr())


@dataclass
class KvPool:
    """Caller-owned paged K/V storage: fp16 [num_pages, kv_heads, page_size, head_dim] each."""
    k: torch.Tensor
    v: torch.Tensor
    desc: L.KvPool

    @property
    def page_size(self):
        return self.desc.page_size


@dataclass
class KvPoolFp8:
    """Caller-owned paged K/V storage in FP8 E4M3FN: uint8 [num_pages, kv_heads, page_size, head_dim] each, one
    scale per tensor (stored byte = encode(x / scale))."""
    k: torch.Tensor
    v: torch.Tensor
    desc: L.KvPoolFp8

    @property
    def page_size(self):
        return self.desc.page_size


@dataclass
class MlaPool:
    """Caller-owned paged latent storage: fp16 [num_pages, page_size, latent_dim + rope_dim]."""
    rows: torch.Tensor
    desc: L.MlaPool


@dataclass
class PageTable:
    pages: torch.Tensor  # int32 [batch, max_pages] on the device
    lens: torch.Tensor   # int32 [batch] on the device
    desc: L.PageTable
    host_pages: Optional[torch.Tensor] = None
    host_lens: Optional[torch.Tensor] = None


class CudaBackend:
    def __init__(self, device: int = 0, stream: Optional[torch.cuda.Stream] = None):
        if not torch.cuda.is_available():
            raise RuntimeError("CudaBackend needs a CUDA device: there is no CPU fallback")
        self._lib = L.load()
        self.device = torch.device("cuda", device)
        torch.cuda.set_device(self.device)
        self.stream = stream if stream is not None else torch.cuda.current_stream(self.device)
        h = C.c_void_p()
        # torch's default stream has handle 0, which the C ABI reads as "make your own": name the legacy
        # default stream explicitly (cudaStreamLegacy == 1) so that torch ops and library ops stay ordered
        rc = self._lib.inf_ctx_create(device, C.c_void_p(self.stream.cuda_stream or 1), C.byref(h))
        if rc != L.INF_OK:
            raise InfernoError(rc, "inf_ctx_create failed (is this an sm_100 GPU?)")
        self._ctx = h
        self._keep = []

    def set_stream(self, stream: torch.cuda.Stream):
        """Enqueue subsequent ops on `stream` (e.g. the capture stream of a CUDA graph)."""
        self._check(self._lib.inf_ctx_set_stream(self._ctx, C.c_void_p(stream.cuda_stream or 1)))
        self.stream = stream

    def capture_graph(self, fn, warmup: int = 2):
        """Run `fn` (a sequence of backend ops with fixed arguments) a few times, then capture it into a CUDA
        graph.  Returns the graph; `graph.replay()` re-launches the whole step with one driver call."""
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        old = self.stream
        with torch.cuda.stream(side):
            self.set_stream(side)
            for _ in range(warmup):
                fn()
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                fn()
        self.set_stream(old)
        torch.cuda.current_stream(self.device).wait_stream(side)
        return graph

    # ------------------------------------------------------------------ multi-GPU
    def comm_unique_id(self) -> bytes:
        buf = C.create_string_buffer(128)
        self._check(self._lib.inf_comm_unique_id(self._ctx, buf))
        return buf.raw

    def comm_init(self, unique_id: bytes, rank: int, nranks: int):
        h = C.c_void_p()
        self._check(self._lib.inf_comm_init(self._ctx, C.create_string_buffer(unique_id, 128), rank, nranks, C.byref(h)))
        self._comm, self._comm_size = h, nranks
        return h

    def allgather_heads(self, local_out: torch.Tensor) -> torch.Tensor:
        """local_out [tokens, heads/N, dim] -> [tokens, heads, dim] through inf_allgather_heads (NCCL)."""
        n = self._comm_size
        t, h, d = local_out.shape
        local_out = local_out.contiguous()
        gathered = torch.empty((n * t, h, d), dtype=local_out.dtype, device=local_out.device)
        rc = self._lib.inf_allgather_heads(self._comm, _ptr(local_out), _ptr(gathered),
                                           local_out.numel() * local_out.element_size())
        self._check(rc)
        return gathered.view(n, t, h, d).permute(1, 0, 2, 3).reshape(t, n * h, d)

    def allgather_into(self, local_out: torch.Tensor, gathered: torch.Tensor) -> torch.Tensor:
        """inf_allgather_heads without any allocation or layout change: `gathered` (contiguous, world x the bytes
        of `local_out`) receives every rank's block in rank order, [world][...local shape...]; the consumer indexes
        the rank-major layout itself."""
        nbytes = local_out.numel() * local_out.element_size()
        assert local_out.is_contiguous() and gathered.is_contiguous()
        assert gathered.numel() * gathered.element_size() == self._comm_size * nbytes
        self._check(self._lib.inf_allgather_heads(self._comm, _ptr(local_out), _ptr(gathered), nbytes))
        return gathered

    def comm_barrier_is_p2p(self) -> bool:
        return bool(self._lib.inf_comm_barrier_is_p2p(self._comm))

    def comm_barrier(self):
        """Stream-ordered barrier over the communicator's ranks (after it, every rank's earlier work has finished)."""
        self._check(self._lib.inf_comm_barrier(self._comm))

    # ---- the all-gather fused into the prefill kernels: peers' copies of the gathered tensor, mapped into this process
    def peer_export(self, t: torch.Tensor) -> bytes:
        """Bytes that let another process of this box map the allocation `t` lives in (its storage must come from
        cudaMalloc, which is what torch's default allocator uses)."""
        buf = C.create_string_buffer(L.PEER_HANDLE_BYTES)
        self._check(self._lib.inf_peer_export(self._ctx, C.c_void_p(t.data_ptr()), buf))
        return buf.raw

    def peer_open(self, handle: bytes) -> int:
        """Device address, valid in this process, of the tensor a peer exported."""
        p = C.c_void_p()
        self._check(self._lib.inf_peer_open(self._ctx, C.create_string_buffer(handle, L.PEER_HANDLE_BYTES), C.byref(p)))
        self._peer_maps = getattr(self, "_peer_maps", [])
        self._peer_maps.append((p.value, handle))
        return p.value

    def peer_close_all(self):
        for ptr, handle in getattr(self, "_peer_maps", []):
            self._lib.inf_peer_close(self._ctx, C.c_void_p(ptr), C.create_string_buffer(handle, L.PEER_HANDLE_BYTES))
        self._peer_maps = []

    @staticmethod
    def _peer_array(peers, byte_offset):
        arr = (C.c_void_p * max(1, len(peers)))(*[C.c_void_p(p + byte_offset) for p in peers])
        return arr

    def comm_destroy(self):
        if getattr(self, "_comm", None):
            self._lib.inf_comm_destroy(self._comm)
            self._comm = None

    def close(self):
        if getattr(self, "_ctx", None):
            self.peer_close_all()
        self.comm_destroy()
        if getattr(self, "_ctx", None):
            self._lib.inf_ctx_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------------ helpers
    def _check(self, rc: int):
        if rc == L.INF_OK:
            return True
        if rc == L.INF_UNSUPPORTED:
            return None  # the reference's Ok(None)
        raise InfernoError(rc, self._lib.inf_last_error(self._ctx).decode())

    def device_values_supported(self) -> bool:  # backend.rs:1060
        return bool(self._lib.inf_device_values_supported(self._ctx))

    def device_flush(self):  # backend.rs:1066
        self._check(self._lib.inf_flush(self._ctx))

    def device_submit(self):  # backend.rs:1072
        self._check(self._lib.inf_submit(self._ctx))

    def device_profile_boundary(self, enable: bool):  # backend.rs:1080
        self._check(self._lib.inf_profile_enable(self._ctx, int(enable)))

    def profile_read(self, kernel_name: str):
        """(summed device milliseconds, launches) of one kernel since the last read."""
        ms, n = C.c_double(), C.c_int32()
        self._check(self._lib.inf_profile_read(self._ctx, kernel_name.encode(), C.byref(ms), C.byref(n)))
        return ms.value, n.value

    def device_upload_f32_tensor(self, host: torch.Tensor) -> torch.Tensor:  # backend.rs:1086
        host = host.contiguous().float()
        out = torch.empty(host.shape, dtype=torch.float32, device=self.device)
        self._check(self._lib.inf_upload(self._ctx, _ptr(out), C.c_void_p(host.data_ptr()), host.numel() * 4))
        return out

    def device_upload_f32_tensor_as_f16(self, host: torch.Tensor) -> torch.Tensor:  # backend.rs:1092
        host = host.contiguous().float()
        out = torch.empty(host.shape, dtype=torch.float16, device=self.device)
        self._check(self._lib.inf_upload_f32_as_f16(self._ctx, _ptr(out), C.c_void_p(host.data_ptr()), host.numel()))
        return out

    def device_download_f32_tensor(self, dev: torch.Tensor) -> torch.Tensor:  # backend.rs:1136
        assert dev.dtype == torch.float32
        out = torch.empty(dev.shape, dtype=torch.float32)
        self._check(self._lib.inf_download(self._ctx, C.c_void_p(out.data_ptr()), _ptr(dev), dev.numel() * 4))
        return out

    # ------------------------------------------------------------------ descriptors
    def prepare_rope_table(self, inv_freq, rotary_dim: int, attention_factor: float) -> L.RopeTable:  # backend.rs:1227
        host = torch.as_tensor(inv_freq, dtype=torch.float32).contiguous()
        t = L.RopeTable()
        self._check(self._lib.inf_rope_table_create(self._ctx, C.c_void_p(host.data_ptr()), host.numel(), rotary_dim,
                                                    attention_factor, C.byref(t)))
        return t

    def prepare_kv_pool(self, num_pages: int, page_size: int, kv_heads: int, head_dim: int = 128) -> KvPool:
        """prepare_laguna_f16_kv_cache (backend.rs:1322) for the paged layout; zero-filled."""
        if page_size <= 0 or page_size % 16:
            raise InfernoError(L.INF_E_CACHE, f"page_size must be a positive multiple of 16, got {page_size}")
        if head_dim != 128:
            raise InfernoError(L.INF_E_SHAPE, f"head_dim must be 128, got {head_dim}")
        k = torch.zeros((num_pages, kv_heads, page_size, head_dim), dtype=torch.float16, device=self.device)
        v = torch.zeros_like(k)
        return KvPool(k, v, L.KvPool(k.data_ptr(), v.data_ptr(), num_pages, page_size, kv_heads, head_dim))

    def prepare_kv_pool_fp8(self, num_pages: int, page_size: int, kv_heads: int, key_scale: float, value_scale: float,
                            head_dim: int = 128) -> KvPoolFp8:
        """prepare_laguna_fp8_kv_cache (crates/backend/src/metal/fp8_attention.rs) for the paged layout; zero-filled."""
        if page_size <= 0 or page_size % 16:
            raise InfernoError(L.INF_E_CACHE, f"page_size must be a positive multiple of 16, got {page_size}")
        if head_dim != 128:
            raise InfernoError(L.INF_E_SHAPE, f"head_dim must be 128, got {head_dim}")
        if not (key_scale > 0 and value_scale > 0):
            raise InfernoError(L.INF_E_CONFIG, "FP8 scales must be positive and finite")
        k = torch.zeros((num_pages, kv_heads, page_size, head_dim), dtype=torch.uint8, device=self.device)
        v = torch.zeros_like(k)
        return KvPoolFp8(k, v, L.KvPoolFp8(k.data_ptr(), v.data_ptr(), num_pages, page_size, kv_heads, head_dim,
                                            key_scale, value_scale))

    def prepare_mla_pool(self, num_pages: int, page_size: int = 64, latent_dim: int = 512, rope_dim: int = 64) -> MlaPool:
        if page_size != 64:
            raise InfernoError(L.INF_E_CACHE, f"MLA page_size must be 64, got {page_size}")
        if latent_dim != 512 or rope_dim != 64:
            raise InfernoError(L.INF_E_SHAPE, "MLA rows must be 512 + 64 wide")
        rows = torch.zeros((num_pages, page_size, latent_dim + rope_dim), dtype=torch.float16, device=self.device)
        return MlaPool(rows, L.MlaPool(rows.data_ptr(), num_pages, page_size, latent_dim, rope_dim))

    def page_table(self, pages, lens, validate_on_host: bool = True) -> PageTable:
        """pages int32 [batch, max_pages], lens int32 [batch]; host or device tensors."""
        pages_t = torch.as_tensor(pages, dtype=torch.int32)
        lens_t = torch.as_tensor(lens, dtype=torch.int32)
        hp = pages_t.cpu().contiguous() if validate_on_host else None
        hl = lens_t.cpu().contiguous() if validate_on_host else None
        dp = pages_t.to(self.device).contiguous()
        dl = lens_t.to(self.device).contiguous()
        desc = L.PageTable(dp.data_ptr(), dl.data_ptr(), dp.shape[0], dp.shape[1],
                           hp.data_ptr() if hp is not None else None, hl.data_ptr() if hl is not None else None)
        return PageTable(dp, dl, desc, hp, hl)

    # ------------------------------------------------------------------ RoPE + append
    def qk_rms_norm_rope_device(self, x, norm_weight, eps, position_offset, table):  # backend.rs:1238
        B, T, H, D = x.shape
        out = torch.empty_like(x)
        ok = self._check(self._lib.inf_qk_rms_norm_rope(self._ctx, _ptr(x), _ptr(norm_weight), eps, position_offset,
                                                        C.byref(table), B, T, H, D, _ptr(out)))
        return out if ok else None

    def laguna_qk_rms_norm_rope_pair_device(self, q, k, q_norm, k_norm, eps, position_offset, table):  # backend.rs:1252
        B, T, Hq, D = q.shape
        Hkv = k.shape[2]
        q_out, k_out = torch.empty_like(q), torch.empty_like(k)
        ok = self._check(self._lib.inf_laguna_qk_rms_norm_rope_pair(
            self._ctx, _ptr(q), _ptr(k), _ptr(q_norm), _ptr(k_norm), eps, position_offset, C.byref(table), B, T, Hq,
            Hkv, D, _ptr(q_out), _ptr(k_out)))
        return (q_out, k_out) if ok else None

    def rope_append_gqa(self, q, k, v, rope, pool: KvPool, table: PageTable, q_norm=None, k_norm=None, eps=1e-6,
                        want_k_f32=False):
        """Fused per-head RMSNorm + half-split RoPE + paged KV append.  Returns roped q (fp16)."""
        B, T, Hq, D = q.shape
        if q.dtype != k.dtype or q.dtype != v.dtype or q.dtype not in (torch.float32, torch.float16):
            raise InfernoError(L.INF_E_DTYPE, "q/k/v must share dtype f32 or f16")
        dt = L.DTYPE_F32 if q.dtype == torch.float32 else L.DTYPE_F16
        q_out = torch.empty((B, T, Hq, D), dtype=torch.float16, device=self.device)
        k_f32 = torch.empty(k.shape, dtype=torch.float32, device=self.device) if want_k_f32 else None
        self._check(self._lib.inf_rope_append_gqa(
            self._ctx, _ptr(q), _ptr(k), _ptr(v), dt, _ptr(q_norm), _ptr(k_norm), eps,
            C.byref(rope) if rope is not None else None, C.byref(pool.desc), C.byref(table.desc), T, Hq, _ptr(q_out),
            _ptr(k_f32)))
        return (q_out, k_f32) if want_k_f32 else q_out

    def rope_append_gqa_fp8(self, q, k, v, rope, pool: KvPoolFp8, table: PageTable, q_norm=None, k_norm=None, eps=1e-6,
                            cur_k=None, cur_v=None):
        """Fused per-head RMSNorm + half-split RoPE + paged append into FP8 pages.  Returns (roped q, roped k, v) as
        fp16: attention reads the call's own tokens at full precision, not through the cache."""
        B, T, Hq, D = q.shape
        if q.dtype != k.dtype or q.dtype != v.dtype or q.dtype not in (torch.float32, torch.float16):
            raise InfernoError(L.INF_E_DTYPE, "q/k/v must share dtype f32 or f16")
        dt = L.DTYPE_F32 if q.dtype == torch.float32 else L.DTYPE_F16
        q_out = torch.empty((B, T, Hq, D), dtype=torch.float16, device=self.device)
        if cur_k is None:
            cur_k = torch.empty(k.shape, dtype=torch.float16, device=self.device)
        if cur_v is None:
            cur_v = torch.empty(v.shape, dtype=torch.float16, device=self.device)
        self._check(self._lib.inf_rope_append_gqa_fp8(
            self._ctx, _ptr(q), _ptr(k), _ptr(v), dt, _ptr(q_norm), _ptr(k_norm), eps,
            C.byref(rope) if rope is not None else None, C.byref(pool.desc), C.byref(table.desc), T, Hq, _ptr(q_out),
            _ptr(cur_k), _ptr(cur_v)))
        return q_out, cur_k, cur_v

    def rope_slice_device(self, x, rope_dim, position_offset, theta):  # backend.rs:1866
        B, T, H, R = x.shape
        out = torch.empty_like(x)
        self._check(self._lib.inf_rope_slice(self._ctx, _ptr(x), _ptr(out), B, T, H, rope_dim, position_offset, theta))
        return out

    def mla_kv_postprocess_device(self, x, norm_weight, eps, theta, pool: MlaPool, table: PageTable, want_outputs=True):
        """mla_kv_postprocess_device (backend.rs:1895) fused with the paged append."""
        B, T, W = x.shape
        lat = torch.empty((B, T, pool.desc.latent_dim), dtype=torch.float32, device=self.device) if want_outputs else None
        rope = torch.empty((B, T, pool.desc.rope_dim), dtype=torch.float32, device=self.device) if want_outputs else None
        self._check(self._lib.inf_mla_kv_postprocess_append(self._ctx, _ptr(x), _ptr(norm_weight), eps, theta,
                                                            C.byref(pool.desc), C.byref(table.desc), T, _ptr(lat),
                                                            _ptr(rope)))
        return lat, rope

    # ------------------------------------------------------------------ attention
    def gqa_decode_paged(self, q_f16, pool: KvPool, table: PageTable, max_len: int, split_chunk: int = 512,
                         sliding_window: int = 0, gate=None, scale: float = 0.0, out_dtype=torch.float32, out=None,
                         peers=None):
        """`peers`: device addresses (peer_open) of the other ranks' copies of the gathered [all sequences, Hq, D]
        output that `out` is this rank's block of rows of: every output row is also stored there."""
        B, Hq, D = q_f16.shape
        if out is None:
            out = torch.empty((B, Hq, D), dtype=out_dtype, device=self.device)
        dt = L.DTYPE_F32 if out.dtype == torch.float32 else L.DTYPE_F16
        if peers is None:
            ok = self._check(self._lib.inf_gqa_decode_paged(self._ctx, _ptr(q_f16), C.byref(pool.desc),
                                                            C.byref(table.desc), Hq, max_len, split_chunk,
                                                            sliding_window, _ptr(gate), scale, _ptr(out), dt))
            return out if ok else None
        assert out.is_contiguous()
        arr = self._peer_array(peers, out.storage_offset() * out.element_size())
        ok = self._check(self._lib.inf_gqa_decode_paged_peers(
            self._ctx, _ptr(q_f16), C.byref(pool.desc), C.byref(table.desc), Hq, max_len, split_chunk, sliding_window,
            _ptr(gate), scale, _ptr(out), dt, arr, len(peers)))
        return out if ok else None

    def gqa_decode_paged_fp8(self, q_f16, cur_k_f16, cur_v_f16, pool: KvPoolFp8, table: PageTable, max_len: int,
                             split_chunk: int = 512, sliding_window: int = 0, gate=None, scale: float = 0.0,
                             out_dtype=torch.float32, out=None):
        """Decode over FP8 pages: table.lens counts the rows cached BEFORE the current token, whose key and value
        are given as fp16 [B, Hkv, D] and enter the softmax at full precision."""
        B, Hq, D = q_f16.shape
        if out is None:
            out = torch.empty((B, Hq, D), dtype=out_dtype, device=self.device)
        dt = L.DTYPE_F32 if out.dtype == torch.float32 else L.DTYPE_F16
        ok = self._check(self._lib.inf_gqa_decode_paged_fp8(
            self._ctx, _ptr(q_f16), _ptr(cur_k_f16), _ptr(cur_v_f16), C.byref(pool.desc), C.byref(table.desc), Hq,
            max_len, split_chunk, sliding_window, _ptr(gate), scale, _ptr(out), dt))
        return out if ok else None

    def gqa_decode_paged_static(self, q_f16, pool: KvPool, table: PageTable, max_len: int, split_chunk: int = 512,
                                sliding_window: int = 0, gate=None, scale: float = 0.0, out=None):
        """gqa_decode_paged for callers that must not allocate device memory while decoding: the split-KV
        partials go to the fixed array inside the library instead of a cudaMalloc'ed workspace.  `out` must be
        supplied by the caller (allocating it here would defeat the purpose); sizes beyond the array raise
        InfernoError(kind 'Config').  Calls that overlap on one GPU race on the shared array."""
        B, Hq, D = q_f16.shape
        if out is None:
            raise InfernoError(L.INF_E_ARG, "gqa_decode_paged_static writes into a caller-provided `out`")
        dt = L.DTYPE_F32 if out.dtype == torch.float32 else L.DTYPE_F16
        ok = self._check(self._lib.inf_gqa_decode_paged_static(self._ctx, _ptr(q_f16), C.byref(pool.desc),
                                                               C.byref(table.desc), Hq, max_len, split_chunk,
                                                               sliding_window, _ptr(gate), scale, _ptr(out), dt))
        return out if ok else None

    def gqa_prefill_paged(self, q_f16, pool: KvPool, table: PageTable, sliding_window: int = 0, gate=None,
                          scale: float = 0.0, out_dtype=torch.float16, out=None, peers=None):
        """`peers`: device addresses (peer_open) of the other ranks' copies of the gathered tensor `out` is a head
        slice of ([B, T, Hq, D] view with the gathered tensor's token stride): every output tile is also stored there."""
        B, T, Hq, D = q_f16.shape
        if out is None:
            out = torch.empty((B, T, Hq, D), dtype=out_dtype, device=self.device)
        dt = L.DTYPE_F32 if out.dtype == torch.float32 else L.DTYPE_F16
        if peers is None:
            ok = self._check(self._lib.inf_gqa_prefill_paged(self._ctx, _ptr(q_f16), C.byref(pool.desc), C.byref(table.desc),
                                                             T, Hq, sliding_window, _ptr(gate), scale, _ptr(out), dt))
            return out if ok else None
        assert out.stride(3) == 1 and out.stride(2) == D and out.stride(0) == T * out.stride(1)
        arr = self._peer_array(peers, out.storage_offset() * out.element_size())
        ok = self._check(self._lib.inf_gqa_prefill_paged_peers(
            self._ctx, _ptr(q_f16), C.byref(pool.desc), C.byref(table.desc), T, Hq, sliding_window, _ptr(gate), scale,
            C.c_void_p(out.data_ptr()), dt, out.stride(1), arr, len(peers)))
        return out if ok else None

    def laguna_gated_gqa_f16_attention_device(self, q, k, v, gate, pool: KvPool, table: PageTable, max_len: int,
                                              sliding_window: int = 0):  # backend.rs:1350
        B, T, Hq, D = q.shape
        out = torch.empty((B, T, Hq, D), dtype=torch.float32, device=self.device)
        ok = self._check(self._lib.inf_laguna_gated_gqa_f16_attention(
            self._ctx, _ptr(q), _ptr(k), _ptr(v), _ptr(gate), C.byref(pool.desc), C.byref(table.desc), T, Hq, max_len,
            sliding_window, _ptr(out)))
        return out if ok else None

    def mla_decode_absorbed(self, q_f16, pool: MlaPool, table: PageTable, max_len: int, scale: float,
                            out_dtype=torch.float32, out=None):
        B, T, H, W = q_f16.shape
        if out is None:
            out = torch.empty((B, T, H, pool.desc.latent_dim), dtype=out_dtype, device=self.device)
        dt = L.DTYPE_F32 if out.dtype == torch.float32 else L.DTYPE_F16
        ok = self._check(self._lib.inf_mla_decode_absorbed(self._ctx, _ptr(q_f16), C.byref(pool.desc),
                                                           C.byref(table.desc), T, H, max_len, scale, _ptr(out), dt))
        return out if ok else None

    def mla_decode_absorbed_selected(self, q_f16, pool: MlaPool, table: PageTable, selected, selected_counts,
                                     scale: float, out_dtype=torch.float32, out=None):
        """Absorbed-MLA decode over the rows listed in `selected` (int32 [B, stride] logical row ids, the first
        selected_counts[b] of each row are used): the attention step of DSA sparse decode with the gather fused in."""
        B, T, H, W = q_f16.shape
        assert T == 1 and selected.dtype == torch.int32 and selected_counts.dtype == torch.int32
        if out is None:
            out = torch.empty((B, 1, H, pool.desc.latent_dim), dtype=out_dtype, device=self.device)
        dt = L.DTYPE_F32 if out.dtype == torch.float32 else L.DTYPE_F16
        ok = self._check(self._lib.inf_mla_decode_absorbed_selected(
            self._ctx, _ptr(q_f16), C.byref(pool.desc), C.byref(table.desc), _ptr(selected), _ptr(selected_counts),
            selected.shape[1], H, scale, _ptr(out), dt))
        return out if ok else None

    def selected_decode_attention_device(self, q, selected_k, selected_v, current_k, current_v, include_current_kv: bool):
        """selected_decode_attention_device (backend.rs:2001): q [B,H,1,D] f32, selected_k/v [B,H,S,D/Dv] f32 or fp16,
        current_k/v [B,H,1,D/Dv] f32 -> [B,H,1,Dv] f32."""
        B, H, T, D = q.shape
        S, Dv = selected_k.shape[2], selected_v.shape[3]
        if selected_k.dtype != selected_v.dtype:
            raise InfernoError(L.INF_E_BACKEND, "device selected decode attention selected KV dtype mismatch")
        if T != 1:
            raise InfernoError(L.INF_E_SHAPE, "device_selected_decode_attention_query_tokens: expected [1]")
        dt = L.DTYPE_F32 if selected_k.dtype == torch.float32 else L.DTYPE_F16
        out = torch.empty((B, H, 1, Dv), dtype=torch.float32, device=self.device)
        ok = self._check(self._lib.inf_selected_decode_attention(
            self._ctx, _ptr(q), _ptr(selected_k), _ptr(selected_v), dt, _ptr(current_k), _ptr(current_v), B, H, S, D, Dv,
            int(include_current_kv), _ptr(out)))
        return out if ok else None

    def selected_sequence_attention_device(self, q, past_k, past_v, current_k, current_v):
        """selected_sequence_attention_device (backend.rs:2015): causal rows over past + current, all f32,
        [B,H,T,D] / [B,H,P,D] layouts -> [B,H,T,Dv]."""
        B, H, T, D = q.shape
        P = past_k.shape[2] if past_k is not None else 0
        Dv = current_v.shape[3]
        out = torch.empty((B, H, T, Dv), dtype=torch.float32, device=self.device)
        ok = self._check(self._lib.inf_selected_sequence_attention(
            self._ctx, _ptr(q), _ptr(past_k) if P else None, _ptr(past_v) if P else None, _ptr(current_k),
            _ptr(current_v), B, H, P, T, D, Dv, _ptr(out)))
        return out if ok else None

    def dsa_scores(self, q, weights, past_keys, current_key, out=None):
        """DSA index scores (dsa_kernels.metal:137): q f32 [B,H,D], weights f32 [B,H], past_keys f32 [B,past,D],
        current_key f32 [B,D] -> f32 [B, past + 1]."""
        B, H, D = q.shape
        past = past_keys.shape[1]
        if out is None:
            out = torch.empty((B, past + 1), dtype=torch.float32, device=self.device)
        self._check(self._lib.inf_dsa_scores(self._ctx, _ptr(q), _ptr(weights), _ptr(past_keys) if past else None,
                                             _ptr(current_key), B, past, H, D, _ptr(out)))
        return out

    def dsa_topk(self, scores, top_k: int, out=None):
        """Ids of the top_k scores of every row, best first, ties by lower id (dsa_kernels.metal:182-393);
        int32 [B, top_k] whose entries beyond the row length are -1 (0xffffffff)."""
        B, n = scores.shape
        if out is None:
            out = torch.empty((B, top_k), dtype=torch.int32, device=self.device)
        ok = self._check(self._lib.inf_dsa_topk(self._ctx, _ptr(scores), B, n, top_k, _ptr(out), out.shape[1]))
        return out if ok else None

    def dsa_index_key_device(self, raw_key, weight, bias, rope_dim: int, position_offset: int, theta: float,
                             eps: float = 1e-6):
        """trait Backend::dsa_index_key_device (backend.rs:2061): raw_key f32 [B,T,D] -> LayerNorm(weight, bias) ->
        interleaved-pair rotary encoding of the first rope_dim values (indexer.rs:174-203); f32 [B,T,D]."""
        B, T, D = raw_key.shape
        out = torch.empty_like(raw_key)
        self._check(self._lib.inf_dsa_index_key(self._ctx, _ptr(raw_key), _ptr(weight), _ptr(bias), B, T, D, rope_dim,
                                                position_offset, theta, eps, _ptr(out)))
        return out

    def dsa_query_weights(self, hidden_states, q_raw, weights_proj, heads: int, head_dim: int, rope_dim: int,
                          position_offset: int, theta: float):
        """First half of dsa_decode_topk_device (dsa_kernels.metal:83-135): hidden_states f32 [B,hidden], q_raw f32
        [B,heads*head_dim], weights_proj f32 [hidden,heads] -> (q f32 [B,heads,head_dim] rotated, weights f32 [B,heads])."""
        B, hidden = hidden_states.shape
        q = torch.empty((B, heads, head_dim), dtype=torch.float32, device=self.device)
        w = torch.empty((B, heads), dtype=torch.float32, device=self.device)
        self._check(self._lib.inf_dsa_query_weights(self._ctx, _ptr(hidden_states), _ptr(q_raw), _ptr(weights_proj), B,
                                                    hidden, heads, head_dim, rope_dim, position_offset, theta, _ptr(q),
                                                    _ptr(w)))
        return q, w

    def dsa_decode_topk_device(self, hidden_states, q_raw, past_index_keys, current_index_key, weights_proj, heads: int,
                               head_dim: int, rope_dim: int, position_offset: int, theta: float, top_k: int):
        """trait Backend::dsa_decode_topk_device (backend.rs:2074): query rotation and head weights, index scores over
        the past keys and the current one, top-k.  hidden_states [B,1,hidden], q_raw [B,1,heads*head_dim],
        past_index_keys [B,past,head_dim], current_index_key [B,1,head_dim]; int32 ids [B, top_k] on the device."""
        B = hidden_states.shape[0]
        q, w = self.dsa_query_weights(hidden_states.reshape(B, -1), q_raw.reshape(B, -1), weights_proj, heads, head_dim,
                                      rope_dim, position_offset, theta)
        scores = self.dsa_scores(q, w, past_index_keys, current_index_key.reshape(B, head_dim))
        return self.dsa_topk(scores, top_k)

    def fp8_e4m3fn_encode(self, x, scale: float):
        """FP8 E4M3FN encode of x / scale (fp8_attention_kernels.metal:29-54): f32 -> uint8, same shape."""
        out = torch.empty(x.shape, dtype=torch.uint8, device=self.device)
        self._check(self._lib.inf_fp8_e4m3fn_encode(self._ctx, _ptr(x), x.numel(), scale, _ptr(out)))
        return out

    def fp8_e4m3fn_decode(self, b, scale: float):
        """FP8 E4M3FN decode times scale (fp8_attention_kernels.metal:11-27): uint8 -> f32, same shape."""
        out = torch.empty(b.shape, dtype=torch.float32, device=self.device)
        self._check(self._lib.inf_fp8_e4m3fn_decode(self._ctx, _ptr(b), b.numel(), scale, _ptr(out)))
        return out

    def kv_pool_from_fp8(self, k_fp8, v_fp8, key_scale: float, value_scale: float, pool: KvPool):
        """FP8 K / V page arrays dequantised into the fp16 pool of the same geometry."""
        self._check(self._lib.inf_kv_pool_from_fp8(self._ctx, _ptr(k_fp8), _ptr(v_fp8), key_scale, value_scale,
                                                   C.byref(pool.desc)))

    def q8_rows_encode(self, x):
        """Q8Row encode (crates/cache/src/cold_kv.rs:1624): f32 [..., dim] -> uint8 [rows, 4 + dim]."""
        dim = x.shape[-1]
        rows = x.numel() // dim
        out = torch.empty((rows, dim + 4), dtype=torch.uint8, device=self.device)
        self._check(self._lib.inf_q8_rows_encode(self._ctx, _ptr(x), rows, dim, _ptr(out)))
        return out

    def q8_rows_decode(self, payload, dim: int):
        """Q8Row decode (cast_kernels.metal:31): uint8 [rows, 4 + dim] -> f32 [rows, dim]."""
        rows = payload.numel() // (dim + 4)
        out = torch.empty((rows, dim), dtype=torch.float32, device=self.device)
        self._check(self._lib.inf_q8_rows_decode(self._ctx, _ptr(payload), rows, dim, _ptr(out)))
        return out

    def mla_pool_thaw_q8_rows(self, latent_payload, rope_payload, pool: MlaPool, table: PageTable, first_token: int,
                              tokens: int):
        """Cold Q8Row latent / rope rows dequantised straight into the pages of the MLA pool."""
        self._check(self._lib.inf_mla_pool_thaw_q8_rows(self._ctx, _ptr(latent_payload), _ptr(rope_payload),
                                                        C.byref(pool.desc), C.byref(table.desc), first_token, tokens))

    def q8_0_packed_heads_matvec(self, weights_u8, x, out_features: int):
        """Per-head Q8_0 matvec (q2_kernels.metal:3146): weights uint8 device tensor, x f32 [rows, heads, in]."""
        rows, heads, in_features = x.shape
        out = torch.empty((rows, heads, out_features), dtype=torch.float32, device=self.device)
        self._check(self._lib.inf_q8_0_packed_heads_matvec(self._ctx, _ptr(weights_u8), _ptr(x), rows, heads,
                                                           in_features, out_features, _ptr(out)))
        return out

    def q8_0_absorbed_mla_device(self, k_b_weights, v_b_weights, q_no_rope, q_rope, current_latent, current_rope,
                                 pool: MlaPool, table: PageTable, qk_head_dim: int, value_dim: int, max_len: int, out=None):
        """q8_0_absorbed_mla_device (backend.rs:1982): returns [B, T, H, value_dim] f32, or None when the pool's
        geometry has no device path.  current_latent / current_rope may be None when the rows are already stored."""
        B, T, H, qn = q_no_rope.shape
        if out is None:
            out = torch.empty((B, T, H, value_dim), dtype=torch.float32, device=self.device)
        ok = self._check(self._lib.inf_q8_0_absorbed_mla(
            self._ctx, _ptr(k_b_weights), _ptr(v_b_weights), _ptr(q_no_rope), _ptr(q_rope), _ptr(current_latent),
            _ptr(current_rope), C.byref(pool.desc), C.byref(table.desc), T, H, qn, value_dim, qk_head_dim, max_len,
            _ptr(out)))
        return out if ok else None

    def causal_sequence_attention_device(self, q, k_nope, k_rope, v, scale: float, out_dtype=torch.float16, out=None,
                                         peers=None):
        """causal_sequence_attention_device (backend.rs:2028) for MLA prefill: q [T,H,dn+dr], k_nope [T,H,dn],
        k_rope [T,dr] shared by the heads (or None), v [T,H,dv]; any token/head strides, unit inner stride."""
        T, H, dqk = q.shape
        dn = k_nope.shape[2]
        dr = dqk - dn
        dv = v.shape[2]
        if out is None:
            out = torch.empty((T, H, dv), dtype=out_dtype, device=self.device)
        dt = L.DTYPE_F32 if out.dtype == torch.float32 else L.DTYPE_F16
        for t in (q, k_nope, v) + ((k_rope,) if k_rope is not None else ()):
            assert t.stride(-1) == 1 and t.dtype == torch.float16
        common = (self._ctx, C.c_void_p(q.data_ptr()), q.stride(0), q.stride(1), C.c_void_p(k_nope.data_ptr()),
                  k_nope.stride(0), k_nope.stride(1), C.c_void_p(k_rope.data_ptr()) if k_rope is not None else None,
                  k_rope.stride(0) if k_rope is not None else 0, C.c_void_p(v.data_ptr()), v.stride(0), v.stride(1), T, H,
                  dn, dr, dv, scale, C.c_void_p(out.data_ptr()), out.stride(0), out.stride(1), dt)
        if peers is None:
            ok = self._check(self._lib.inf_mla_prefill_causal(*common))
        else:
            # `out` is this rank's head slice of a gathered [T, all heads, dv] tensor; peers are the other ranks' copies
            arr = self._peer_array(peers, out.storage_offset() * out.element_size())
            ok = self._check(self._lib.inf_mla_prefill_causal_peers(*common, arr, len(peers)))
        return out if ok else None

    def paged_decode_attention_resident_device(self, q, paged_k, cur_k, paged_v, cur_v, past_tokens: int, page_size: int):
        """paged_decode_attention_resident_device (backend.rs:1966): GLM MHA decode, q/cur_k [B,H,D] f32,
        cur_v [B,H,Dv] f32, caches fp16 [pages,B,H,P,D] / [pages,B,H,P,Dv] in identity page order."""
        B, H, D = q.shape
        Dv = cur_v.shape[-1]
        out = torch.empty((B, H, Dv), dtype=torch.float32, device=self.device)
        ok = self._check(self._lib.inf_paged_decode_attention_resident(
            self._ctx, _ptr(q), _ptr(paged_k) if paged_k is not None else None, _ptr(cur_k),
            _ptr(paged_v) if paged_v is not None else None, _ptr(cur_v), B, H, past_tokens, page_size, D, Dv, _ptr(out)))
        return out if ok else None

    def paged_kv_contiguous_device(self, which: torch.Tensor, pool: KvPool, table: PageTable, tokens: int):
        """paged_kv_contiguous_device (backend.rs:2040): gather [batch, kv_heads, tokens, head_dim] out of the pages."""
        B = table.desc.batch
        out = torch.empty((B, pool.desc.kv_heads, tokens, pool.desc.head_dim), dtype=torch.float16, device=self.device)
        self._check(self._lib.inf_linearize_paged(self._ctx, _ptr(which), C.byref(pool.desc), C.byref(table.desc),
                                                  tokens, _ptr(out)))
        return out
