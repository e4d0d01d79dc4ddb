"""The kernel backend: thin, shape-checking wrappers around the sm_100a launchers.

There is no other backend in the package and no fallback: constructing
``NativeOps`` without a CUDA device, or without a kernel library that builds and
loads, raises.  Every method takes and returns torch tensors on the CUDA device;
outputs are allocated with torch's caching allocator (which is also what makes
the calls capturable in a CUDA graph).
"""
from __future__ import annotations

import os

import torch

from ..build import load_kernels

_F32, _BF16 = 0, 1


def _dt(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return _F32
    if dtype == torch.bfloat16:
        return _BF16
    raise TypeError(f"kernels take float32 or bfloat16, got {dtype}")


def _p(t: torch.Tensor | None) -> int:
    return 0 if t is None else t.data_ptr()


class KernelError(RuntimeError):
    pass


class _Branch:
    """A piece of a step that may run beside the launching stream.  ``with branch:`` launches
    what is inside on a second stream that starts after everything launched so far;
    ``branch.join()`` makes the launching stream wait for it.  Inactive, it does nothing and the
    work stays in order on the launching stream."""

    def __init__(self, side):
        self.side = side
        self.main = None
        self.ctx = None

    def __enter__(self):
        if self.side is not None:
            self.main = torch.cuda.current_stream()
            self.side.wait_stream(self.main)
            self.ctx = torch.cuda.stream(self.side)
            self.ctx.__enter__()
        return self

    def __exit__(self, *exc):
        if self.ctx is not None:
            self.ctx.__exit__(*exc)
            self.ctx = None
        return False

    def join(self):
        if self.side is not None and self.main is not None:
            self.main.wait_stream(self.side)


class NativeOps:
    """``fast=False`` keeps every product and the attention on the plain FMA kernels
    (the path the 32-bit mode always takes)."""

    def __init__(self, fast: bool = True):
        if not torch.cuda.is_available():
            raise KernelError("dlm_b200 needs a CUDA device: there is no CPU path")
        self.k = load_kernels()
        self.fast = 1 if fast else 0
        self.launches = 0        # kernels launched through this object (for the benchmark's count)
        self.tc = bool(self.k.gemm_tc_enabled()) if fast else False
        self.branches = os.environ.get("DLM_B200_NO_BRANCH", "") in ("", "0")
        self._side = None        # second stream for branches of a step (made at first use)

    @staticmethod
    def _stream() -> int:
        return torch.cuda.current_stream().cuda_stream

    def branch(self, rows: int) -> _Branch:
        """A branch for work on ``rows`` tokens that is independent of what the caller launches
        next.  With few rows the kernels stream weights and leave most of the machine idle
        between them, so two chains side by side fill it better; with many rows each kernel
        fills the machine alone and the branch stays inactive."""
        if not self.fast or rows > 64 or not self.branches:
            return _Branch(None)
        if self._side is None:
            self._side = torch.cuda.Stream()
        return _Branch(self._side)

    def check_errors(self) -> None:
        """Raises if a kernel refused an access (page or token id outside its table)."""
        flag = self.k.take_error_flag()
        if flag == 5:
            # a kernel gave up on a wait: the decode attention's split counters may not be back at zero
            self.k.reset_decode_merge_counters(self._stream())
        if flag:
            what = {1: "token id outside the vocabulary", 2: "cache slot outside the pool",
                    3: "a visible key has no page", 4: "expert id outside the table",
                    5: "a wait inside a kernel ran out (copy or tensor-core pipeline)"}.get(flag, "unknown")
            raise KernelError(f"a kernel reported error {flag}: {what}")

    # ----------------------------------------------------------------- basic
    def embed(self, tokens, table):
        T, (V, H) = tokens.numel(), table.shape
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
        self.launches += 1
        self.k.embed(_p(tokens), _p(table), _p(out), T, H, V, _dt(table.dtype), self._stream())
        return out

    def rmsnorm(self, x, w, eps, out_dtype, rows=None):
        H = x.shape[-1]
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, H), dtype=out_dtype, device=x.device)
        self.launches += 1
        self.k.rmsnorm(_p(x), _p(w), _p(out), _p(rows), n, H, float(eps), _dt(out_dtype), self._stream())
        return out

    # -------------------------------------------------------------- products
    def _gemm(self, a, w, out, M, N, K, epilogue, *, bias=None, a_rows=None, offsets=None, num_experts=0,
              w_expert_stride=0, ldo=None):
        self.launches += 1
        self.k.gemm(_p(a), a.stride(0), _p(a_rows), _p(w), K, w_expert_stride, _p(offsets), num_experts, _p(bias),
                    _p(out), out.stride(0) if ldo is None else ldo, M, N, K, _dt(a.dtype), _dt(out.dtype), epilogue,
                    self.fast, self._stream())

    def linear(self, a, w, bias, out_dtype):
        (M, K), N = a.shape, w.shape[0]
        assert w.shape[1] == K and a.dtype == w.dtype
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        self._gemm(a, w, out, M, N, K, self.k.EPI_STORE, bias=bias)
        return out

    def linear_add(self, a, w, resid):
        (M, K), N = a.shape, w.shape[0]
        assert w.shape[1] == K and resid.shape == (M, N) and resid.dtype == torch.float32
        self._gemm(a, w, resid, M, N, K, self.k.EPI_ADD)

    def linear_swiglu(self, a, w_gate_up):
        (M, K), N = a.shape, w_gate_up.shape[0]
        out = torch.empty((M, N // 2), dtype=a.dtype, device=a.device)
        self._gemm(a, w_gate_up, out, M, N, K, self.k.EPI_SWIGLU)
        return out

    def grouped_swiglu(self, a, w_gate_up, offsets, rows):
        E, N, K = w_gate_up.shape
        M = rows.numel()
        out = torch.empty((M, N // 2), dtype=a.dtype, device=a.device)
        if (self.fast and self.tc and a.dtype == torch.bfloat16 and 8 * M > 9 * E and K % 8 == 0
                and a.stride(0) == K):
            # more than about a row per expert (the kernels' own rule): put each expert's rows side by side, so that the TMA can fetch them as tiles
            gathered = torch.empty((M, K), dtype=a.dtype, device=a.device)
            self.launches += 1
            self.k.gather_rows(_p(a), _p(rows), _p(gathered), M, K, _dt(a.dtype), self._stream())
            self._gemm(gathered, w_gate_up, out, M, N, K, self.k.EPI_SWIGLU, offsets=offsets, num_experts=E,
                       w_expert_stride=N * K)
            return out
        self._gemm(a, w_gate_up, out, M, N, K, self.k.EPI_SWIGLU, a_rows=rows, offsets=offsets, num_experts=E,
                   w_expert_stride=N * K)
        return out

    def grouped_linear(self, a, w, offsets):
        E, N, K = w.shape
        M = a.shape[0]
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
        self._gemm(a, w, out, M, N, K, self.k.EPI_STORE, offsets=offsets, num_experts=E, w_expert_stride=N * K)
        return out

    # ------------------------------------------------------------- attention
    def rope_kv_write(self, qkv, positions, inv_freq, rotary_dim, slots, k_cache, v_cache, nh, nkv, hd, out_dtype,
                      interleaved=False):
        """``interleaved``: rotary pairs are dims (2i, 2i + 1) instead of (i, i + rotary_dim / 2)."""
        T = qkv.shape[0]
        assert qkv.dtype == torch.float32 and qkv.shape[1] == (nh + 2 * nkv) * hd
        total_pages, nkv_c, page_size, hd_c = k_cache.shape
        assert (nkv_c, hd_c) == (nkv, hd) and k_cache.dtype == out_dtype
        q = torch.empty((T, nh * hd), dtype=out_dtype, device=qkv.device)
        self.launches += 1
        self.k.rope_kv_write(_p(qkv), _p(positions), _p(inv_freq), int(rotary_dim), int(bool(interleaved)), _p(slots),
                             _p(q), _p(k_cache),
                             _p(v_cache), T, nh, nkv, hd, page_size, total_pages, _dt(out_dtype), self._stream())
        return q

    def attention(self, q, k_cache, v_cache, block_table, cu_q, kv_len, window, scale, nh, nkv, hd, max_q_len,
                  max_kv_len, num_single=0):
        T = q.shape[0]
        R, width = block_table.shape
        total_pages, _, page_size, _ = k_cache.shape
        out = torch.empty_like(q)
        scratch = None
        if self.fast and num_single > 0:
            n = self.k.attention_scratch_floats(R, nh, nkv, hd, int(max_kv_len))
            if n > 0:
                scratch = torch.empty((n,), dtype=torch.float32, device=q.device)
        # the tensor-core decode kernel merges its key splits itself; the FMA one has a merge kernel behind it
        decode_kernels = 1 if (q.dtype == torch.bfloat16 and hd in (16, 32, 48, 64, 96, 128)) else 2
        self.launches += 1 if scratch is None else (decode_kernels if num_single == R else decode_kernels + 1)
        self.k.attention(_p(q), _p(k_cache), _p(v_cache), _p(block_table), width, _p(cu_q), _p(kv_len), _p(out), T, R,
                         nh, nkv, hd, page_size, total_pages, int(window), float(scale), int(max_q_len),
                         int(max_kv_len), int(num_single), _p(scratch), _dt(q.dtype), self.fast, self._stream())
        return out

    # ------------------------------------------------------------------- moe
    def router_topk(self, h, w, E, k, norm, has_gate, norm_weight=None, eps=0.0, score="softmax", scale=1.0,
                    select_bias=None):
        """Scores (``score``: softmax over the experts, or a sigmoid of each logit), the k best (chosen on
        score + ``select_bias`` when that is given), optionally renormalised, times ``scale``.  ``h`` is one
        of: activations in the weights' dtype; the 32-bit residual together with ``norm_weight`` / ``eps``
        (the RMS norm then runs inside the kernel, in 32-bit); 32-bit activations that are already normalised."""
        T, H = h.shape
        assert w.shape == (E + (1 if has_gate else 0), H)
        assert h.dtype in (w.dtype, torch.float32) and (norm_weight is None or h.dtype == torch.float32)
        score_fn = {"softmax": 0, "sigmoid": 1}[score]
        h_is_f32 = int(norm_weight is None and h.dtype == torch.float32 and w.dtype != torch.float32)
        ids = torch.empty((T, k), dtype=torch.int32, device=h.device)
        wts = torch.empty((T, k), dtype=torch.float32, device=h.device)
        gate = torch.empty((T,), dtype=torch.float32, device=h.device) if has_gate else None
        logits = torch.empty((T, w.shape[0]), dtype=torch.float32, device=h.device)
        self.launches += 2
        self.k.router_topk(_p(h), _p(w), _p(norm_weight), float(eps), _p(logits), _p(ids), _p(wts), _p(gate), T, H,
                           E, k, int(norm), int(has_gate), _dt(w.dtype), h_is_f32, score_fn, float(scale),
                           _p(select_bias), self._stream())
        return ids, wts, gate

    def route(self, h, w, E, k, norm, has_gate, norm_weight=None, eps=0.0, score="softmax", scale=1.0,
              select_bias=None, input_settled=False):
        """``router_topk`` and ``moe_permute`` together: ``(ids, wts, gate, offsets, rows, dest)``.  A step
        of at most 48 tokens does all of it in one launch.  ``input_settled``: ``h`` was not written by the
        kernel launched just before this call (it is a step's residual and a norm kernel ran in between); a
        step of few tokens then works its logits out while that kernel ends."""
        T, H = h.shape
        assert w.shape == (E + (1 if has_gate else 0), H)
        assert h.dtype in (w.dtype, torch.float32) and (norm_weight is None or h.dtype == torch.float32)
        score_fn = {"softmax": 0, "sigmoid": 1}[score]
        h_is_f32 = int(norm_weight is None and h.dtype == torch.float32 and w.dtype != torch.float32)
        dev = h.device
        ids = torch.empty((T, k), dtype=torch.int32, device=dev)
        wts = torch.empty((T, k), dtype=torch.float32, device=dev)
        gate = torch.empty((T,), dtype=torch.float32, device=dev) if has_gate else None
        logits = torch.empty((T, w.shape[0]), dtype=torch.float32, device=dev)
        offsets = torch.empty((E + 1,), dtype=torch.int32, device=dev)
        rows = torch.empty((T * k,), dtype=torch.int32, device=dev)
        dest = torch.empty((T, k), dtype=torch.int32, device=dev)
        self.launches += self.k.router_topk_permute(_p(h), _p(w), _p(norm_weight), float(eps), _p(logits), _p(ids), _p(wts), _p(gate),
                                   _p(offsets), _p(rows), _p(dest), T, H, E, k, int(norm), int(has_gate),
                                   _dt(w.dtype), h_is_f32, score_fn, float(scale), _p(select_bias),
                                                   int(bool(input_settled)), self._stream())
        return ids, wts, gate, offsets, rows, dest

    def moe_permute(self, ids, E):
        T, k = ids.shape
        n = T * k
        offsets = torch.empty((E + 1,), dtype=torch.int32, device=ids.device)
        rows = torch.empty((n,), dtype=torch.int32, device=ids.device)
        dest = torch.empty((T, k), dtype=torch.int32, device=ids.device)
        self.launches += 1
        self.k.moe_permute(_p(ids), n, k, E, _p(offsets), _p(rows), _p(dest), self._stream())
        return offsets, rows, dest

    def moe_combine(self, y, dest, wts, shared, gate, resid):
        T, H = resid.shape
        self.launches += 1
        self.k.moe_combine(_p(y), _p(dest), _p(wts), _p(shared), _p(gate), _p(resid), T, H, dest.shape[1],
                           self._stream())

    # -------------------------------------------------------------- sampling
    def argmax(self, logits):
        N, V = logits.shape
        out = torch.empty((N,), dtype=torch.int32, device=logits.device)
        nbytes = self.k.argmax_scratch_bytes(N, V)
        scratch = torch.empty((nbytes,), dtype=torch.uint8, device=logits.device) if nbytes else None
        self.launches += 2 if nbytes else 1
        self.k.argmax(_p(logits), _p(out), N, V, _p(scratch), self._stream())
        return out

    def sample(self, logits, params, top_k, u, seen_offsets, seen_tokens):
        N, V = logits.shape
        out = torch.empty((N,), dtype=torch.int32, device=logits.device)
        scratch = torch.empty((N, V), dtype=torch.float32, device=logits.device)
        self.launches += 1
        self.k.sample(_p(logits), _p(out), N, V, _p(params), _p(top_k), _p(u), _p(seen_offsets), _p(seen_tokens),
                      _p(scratch), self._stream())
        return out
