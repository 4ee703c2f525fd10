"""Python mirror of the operator front-end (`tensor_<op>` names of anyGPU's srcs/ops, srcs/fused, srcs/models/zamba2)
over the C ABI. torch tensors are used purely as owners of device memory; every computation happens in
libanygpu_b200.so. Raises if the tensors are not CUDA tensors or the library is missing: there is no CPU path.

The C++ header layer in include/anygpu/ is the drop-in for anyGPU itself; this module exists so that the
benchmark and the parity tests can drive the same ABI from Python.
"""
import ctypes

import torch

from . import capi
from .capi import F16, F32, W_KN, W_NK, Mamba2Config, Mamba2Weights

_DT = {torch.float16: F16, torch.float32: F32}


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    if t is None:
        return None
    assert t.is_cuda, "device tensors only: this library has no CPU path"
    return ctypes.c_void_p(t.data_ptr())


def _dt(t):
    return _DT[t.dtype]


def _rows_contig(t):
    assert t.stride(-1) == 1, "innermost dimension must be contiguous"


def _workspace(nbytes, device):
    # torch's caching allocator hands out 512-byte aligned blocks
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


def tensor_linear(xt, wt, w_layout=W_KN, out=None):
    """tensor_linear(xt (*, in), wt (in, out)) of srcs/ops/mm_ops.hpp:206-232. w_layout=W_NK takes wt as (out, in)."""
    K = xt.shape[-1]
    N = wt.shape[1] if w_layout == W_KN else wt.shape[0]
    assert (wt.shape[0] if w_layout == W_KN else wt.shape[1]) == K and wt.is_contiguous()
    x2 = xt.reshape(-1, K)
    _rows_contig(x2)
    M = x2.shape[0]
    if out is None:
        out = torch.empty(xt.shape[:-1] + (N,), dtype=xt.dtype, device=xt.device)
    y2 = out.view(-1, N) if out.dim() != 2 else out
    capi.call("b200_linear", _dt(xt), _p(x2), x2.stride(0) if M > 1 else K, _p(wt), w_layout, _p(y2),
              y2.stride(0) if M > 1 else N, M, K, N, _stream())
    return out


def tensor_mm(lhs, rhs):
    """tensor_mm(lhs (m,k), rhs (k,n)) of srcs/ops/mm_ops.hpp:48-97."""
    return tensor_linear(lhs, rhs)


def tensor_causal_conv1d(xt, wt, bt):
    """tensor_causal_conv1d(xt (batch, dims, seq_len), wt (dims, width), bt (dims)) of srcs/fused/causal_conv1d.hpp:90-117."""
    assert xt.dim() == 3 and xt.is_contiguous() and wt.is_contiguous() and bt.is_contiguous()
    assert xt.shape[1] == wt.shape[0] == bt.shape[0]
    yt = torch.empty_like(xt)
    capi.call("b200_causal_conv1d", _dt(xt), _p(xt), _p(wt), _p(bt), _p(yt), xt.shape[0], xt.shape[1], xt.shape[2],
              wt.shape[1], _stream())
    return yt


def tensor_causal_conv1d_tokens(xt, wt, bt, initial_state=None, want_final_state=False):
    """Token-major variant: xt (batch, seq_len, dims), possibly a slice of a wider tensor (row stride > dims)."""
    assert xt.dim() == 3 and xt.stride(2) == 1 and xt.stride(0) == xt.shape[1] * xt.stride(1)
    b, l, d = xt.shape
    yt = torch.empty((b, l, d), dtype=xt.dtype, device=xt.device)
    fin = torch.empty((b, d, wt.shape[1] - 1), dtype=xt.dtype, device=xt.device) if want_final_state else None
    capi.call("b200_causal_conv1d_tokens", _dt(xt), _p(xt), xt.stride(1), _p(wt), _p(bt), _p(yt), d, _p(initial_state), _p(fin),
              b, l, d, wt.shape[1], _stream())
    return (yt, fin) if want_final_state else yt


def tensor_causal_conv1d_update(x_t, conv_state, wt, bt):
    """One decode step; conv_state (batch, dims, width-1) is advanced in place. x_t (batch, dims), row stride free."""
    assert x_t.dim() == 2 and x_t.stride(1) == 1 and conv_state.is_contiguous()
    b, d = x_t.shape
    y = torch.empty((b, d), dtype=x_t.dtype, device=x_t.device)
    capi.call("b200_causal_conv1d_update", _dt(x_t), _p(x_t), x_t.stride(0), _p(conv_state), _p(wt), _p(bt), _p(y), d, b, d,
              wt.shape[1], _stream())
    return y


def tensor_zamba_gated_rmsnorm(xt, zt, wt, gsize, eps, honor_gsize=False):
    """tensor_zamba_gated_rmsnorm(xt, zt, wt, gsize, eps) of srcs/models/zamba2/zamba_gated_rmsnorm.hpp:9-23.
    Like the reference, the statistic spans the whole last axis whatever gsize says; honor_gsize=True normalises
    per group of gsize elements instead (true Mamba2 behaviour for ngroups > 1)."""
    d = xt.shape[-1]
    x2, z2 = xt.reshape(-1, d) if xt.is_contiguous() else xt, zt.reshape(-1, d) if zt.is_contiguous() else zt
    assert x2.dim() == 2 and z2.dim() == 2
    _rows_contig(x2), _rows_contig(z2)
    rows = x2.shape[0]
    y = torch.empty((rows, d), dtype=xt.dtype, device=xt.device)
    capi.call("b200_gated_rmsnorm", _dt(xt), _p(x2), x2.stride(0), _p(z2), z2.stride(0), _p(wt), _p(y), d, rows, d,
              gsize if honor_gsize else d, float(eps), _stream())
    return y.view(xt.shape) if xt.is_contiguous() else y


def tensor_rms_norm(xt, wt, eps, zero_centered=False):
    """tensor_rms_norm over the last axis (srcs/ops/norm_ops.hpp:134-228): x * rsqrt(mean(x^2) + eps) * (w + zero_centered)."""
    d = xt.shape[-1]
    x2 = xt.reshape(-1, d)
    _rows_contig(x2)
    assert wt.is_contiguous() and wt.numel() == d
    y = torch.empty((x2.shape[0], d), dtype=xt.dtype, device=xt.device)
    capi.call("b200_rms_norm", _dt(xt), _p(x2), x2.stride(0), _p(wt), _p(y), d, x2.shape[0], d, float(eps), int(zero_centered),
              _stream())
    return y.reshape(xt.shape)


def _tok_stride(t, inner):
    """Element stride between tokens of a [b, l, ...] tensor whose trailing dims are dense."""
    assert t.stride(-1) == 1
    st = t.stride(1)
    assert t.stride(0) == t.shape[1] * st, "batch stride must equal seqlen * token stride"
    assert st >= inner
    return st


def tensor_mamba_chunk_scan_combined(x, dt, A, B, C, chunk_size, D=None, dt_bias=None, initial_states=None, a_is_log=False,
                                     exact_final_state=False, final_states_out=None):
    """Argument order of mamba_chunk_scan_combined_ref (scripts/zamba2/mamba_chunk_scan_comb.py:167-172), dt_softplus on.
    x (b,l,H,P), dt (b,l,H), A (H) fp32, B/C (b,l,G,N), D (H) fp32, dt_bias (H) fp32, initial_states (b,H,P,N) fp32.
    Returns (y (b,l,H,P), final_states (b,H,P,N) fp32). When l is not a multiple of chunk_size, final_states follows the
    reference script (padded positions decay it) unless exact_final_state is set (state after the last real token).
    final_states_out: where to write final_states (may be the initial_states tensor itself)."""
    b, l, H, P = x.shape
    G, N = B.shape[2], B.shape[3]
    y = torch.empty((b, l, H, P), dtype=x.dtype, device=x.device)
    fs = final_states_out if final_states_out is not None else torch.empty((b, H, P, N), dtype=torch.float32, device=x.device)
    assert fs.dtype == torch.float32 and fs.is_contiguous() and tuple(fs.shape) == (b, H, P, N)
    lib = capi.load()
    nbytes = lib.b200_mamba_chunk_scan_combined_workspace_bytes(b, l, H, P, G, N, chunk_size)
    ws = _workspace(nbytes, x.device)
    for t in (A, D, dt_bias, initial_states):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous())
    capi.call("b200_mamba_chunk_scan_combined", _dt(x), _p(x), _tok_stride(x, H * P), _p(dt), _tok_stride(dt, H), _p(A),
              int(a_is_log), _p(B), _tok_stride(B, G * N), _p(C), _tok_stride(C, G * N), _p(D), _p(dt_bias), _p(initial_states),
              _p(y), H * P, _p(fs), b, l, H, P, G, N, chunk_size, 2 if exact_final_state else 1, _p(ws), ws.numel(), _stream())
    return y, fs


def tensor_mamba_selective_state_update(ssm_state, x, dt, A, B, C, D=None, dt_bias=None, a_is_log=False):
    """One decode step of the recurrence; ssm_state (b,H,P,N) fp32 is advanced in place. x (b,H,P), dt (b,H), B/C (b,G,N)."""
    b, H, P = x.shape
    G, N = B.shape[1], B.shape[2]
    assert ssm_state.dtype == torch.float32 and ssm_state.is_contiguous()
    y = torch.empty((b, H, P), dtype=x.dtype, device=x.device)
    capi.call("b200_selective_state_update", _dt(x), _p(ssm_state), _p(x), x.stride(0), _p(dt), dt.stride(0), _p(A), int(a_is_log),
              _p(B), B.stride(0), _p(C), C.stride(0), _p(D), _p(dt_bias), _p(y), H * P, b, H, P, G, N, 1, _stream())
    return y


class ZambaMamba2weights:
    """Weights of one Mamba2 mixer, in the style of anyGPU's Zamba2 weight structs (srcs/models/zamba2/zamba_mlp.hpp:13-48).
    Projection weights are (in_features, out_features) as tensor_linear expects unless *_layout says W_NK."""

    def __init__(self, in_proj_weight, conv1d_weight, conv1d_bias, dt_bias, A_log, D, norm_weight, out_proj_weight,
                 in_proj_layout=W_KN, out_proj_layout=W_KN):
        self.in_proj_weight, self.conv1d_weight, self.conv1d_bias = in_proj_weight, conv1d_weight, conv1d_bias
        self.dt_bias, self.A_log, self.D = dt_bias.float().contiguous(), A_log.float().contiguous(), D.float().contiguous()
        self.norm_weight, self.out_proj_weight = norm_weight, out_proj_weight
        self.in_proj_layout, self.out_proj_layout = in_proj_layout, out_proj_layout

    @classmethod
    def from_numpy(cls, w, dtype, device="cuda", layout=W_KN):
        """w: dict of fp32 numpy arrays with (in,out) projection weights (anygpu_b200.synth.make_weights)."""
        t = lambda a, dt: torch.from_numpy(a).to(device=device, dtype=dt).contiguous()
        proj = (lambda a: t(a, dtype)) if layout == W_KN else (lambda a: t(a.T.copy(), dtype))
        return cls(proj(w["in_proj_weight"]), t(w["conv1d_weight"], dtype), t(w["conv1d_bias"], dtype),
                   t(w["dt_bias"], torch.float32), t(w["A_log"], torch.float32), t(w["D"], torch.float32),
                   t(w["norm_weight"], dtype), proj(w["out_proj_weight"]), layout, layout)

    def c_struct(self):
        return Mamba2Weights(self.in_proj_weight.data_ptr(), self.conv1d_weight.data_ptr(), self.conv1d_bias.data_ptr(),
                             self.dt_bias.data_ptr(), self.A_log.data_ptr(), self.D.data_ptr(), self.norm_weight.data_ptr(),
                             self.out_proj_weight.data_ptr(), self.in_proj_layout, self.out_proj_layout)


class ZambaMambaCache:
    """conv_state (b, conv_dim, d_conv-1) in the activation dtype and ssm_state (b,H,P,N) fp32; fills the role of the
    empty ZambaKVcache (srcs/models/zamba2/zamba_sdpa.hpp:13) for the Mamba layers."""

    def __init__(self, conv_state, ssm_state):
        self.conv_state, self.ssm_state = conv_state, ssm_state

    @classmethod
    def zeros(cls, cfg, batch, dtype, device="cuda"):
        conv_dim = cfg["d_inner"] + 2 * cfg["ngroups"] * cfg["d_state"]
        return cls(torch.zeros((batch, conv_dim, cfg["d_conv"] - 1), dtype=dtype, device=device),
                   torch.zeros((batch, cfg["nheads"], cfg["headdim"], cfg["d_state"]), dtype=torch.float32, device=device))


def make_config(cfg):
    return Mamba2Config(cfg["d_model"], cfg["d_inner"], cfg["nheads"], cfg["headdim"], cfg["d_state"], cfg["ngroups"],
                        cfg["d_conv"], cfg["chunk"], cfg.get("norm_group_size") or 0, cfg["eps"])


class Mamba2Mixer:
    """Holds config, weights and a preallocated workspace; `prefill` / `decode` are single C-ABI calls."""

    def __init__(self, cfg, weights):
        self.cfg, self.w = cfg, weights
        self.c_cfg, self.c_w = make_config(cfg), weights.c_struct()
        self.dtype = weights.in_proj_weight.dtype
        self.device = weights.in_proj_weight.device
        self._ws = None

    def _ensure_ws(self, nbytes):
        if self._ws is None or self._ws.numel() < nbytes:
            self._ws = _workspace(nbytes, self.device)
        return self._ws

    def prefill(self, u, cache=None, initial_states=None, out=None):
        """tensor_zamba_mamba2_mixer for a whole sequence: u (b,l,d_model) -> (b,l,d_model). Fills `cache` when given."""
        b, l, _ = u.shape
        assert u.is_contiguous() and u.dtype == self.dtype
        lib = capi.load()
        ws = self._ensure_ws(lib.b200_mamba2_mixer_prefill_workspace_bytes(ctypes.byref(self.c_cfg), _DT[self.dtype], b, l))
        if out is None:
            out = torch.empty_like(u)
        capi.call("b200_mamba2_mixer_prefill", _DT[self.dtype], ctypes.byref(self.c_cfg), ctypes.byref(self.c_w), _p(u), _p(out),
                  b, l, _p(initial_states), _p(cache.conv_state) if cache else None, _p(cache.ssm_state) if cache else None,
                  _p(ws), ws.numel(), _stream())
        return out

    def prefill_continue(self, u, cache, out=None):
        """`u` (b,l,d_model) are the next l tokens of sequences whose state so far is in `cache` (zeros for new sequences);
        the cache is advanced in place. Feeding a prompt piece by piece equals one prefill over the whole prompt."""
        b, l, _ = u.shape
        assert u.is_contiguous() and u.dtype == self.dtype
        lib = capi.load()
        ws = self._ensure_ws(lib.b200_mamba2_mixer_prefill_continue_workspace_bytes(ctypes.byref(self.c_cfg), _DT[self.dtype], b, l))
        if out is None:
            out = torch.empty_like(u)
        capi.call("b200_mamba2_mixer_prefill_continue", _DT[self.dtype], ctypes.byref(self.c_cfg), ctypes.byref(self.c_w), _p(u),
                  _p(out), b, l, _p(cache.conv_state), _p(cache.ssm_state), _p(ws), ws.numel(), _stream())
        return out

    def prefill_varlen(self, u, cu_seqlens, initial_states=None, cache=None, out=None):
        """Packed batch: `u` (total_tokens, d_model) holds len(cu_seqlens)-1 sequences back to back, sequence s in rows
        cu_seqlens[s]:cu_seqlens[s+1] (host integers). `cache`, if given, has one entry per sequence and receives the final
        states. Each sequence gets what prefill() gives for it alone."""
        cu = [int(v) for v in cu_seqlens]
        nseq = len(cu) - 1
        total = cu[-1]
        assert u.is_contiguous() and u.dtype == self.dtype and u.shape[0] == total
        lib = capi.load()
        ws = self._ensure_ws(max(1, lib.b200_mamba2_mixer_prefill_varlen_workspace_bytes(ctypes.byref(self.c_cfg), _DT[self.dtype], total)))
        if out is None:
            out = torch.empty_like(u)
        cu_arr = (ctypes.c_int64 * (nseq + 1))(*cu)
        capi.call("b200_mamba2_mixer_prefill_varlen", _DT[self.dtype], ctypes.byref(self.c_cfg), ctypes.byref(self.c_w), _p(u), _p(out),
                  cu_arr, nseq, _p(initial_states), _p(cache.conv_state) if cache else None, _p(cache.ssm_state) if cache else None,
                  _p(ws), ws.numel(), _stream())
        return out

    def prefill_host(self, u_host, out_host, overlap=False):
        """Same with HOST (pinned) tensors: H2D copy, mixer, D2H copy, all inside the one C-ABI call. overlap=True vouches
        that the call needs nothing queued on the stream since the previous call (u_host filled by the CPU, weights untouched),
        which lets a call run under the copy-out of the call before it (B200_HOST_OVERLAP)."""
        b, l, _ = u_host.shape
        assert not u_host.is_cuda and not out_host.is_cuda and u_host.is_contiguous() and out_host.is_contiguous()
        lib = capi.load()
        ws = self._ensure_ws(lib.b200_mamba2_mixer_prefill_host_workspace_bytes(ctypes.byref(self.c_cfg), _DT[self.dtype], b, l))
        capi.call("b200_mamba2_mixer_prefill_host_ex", _DT[self.dtype], ctypes.byref(self.c_cfg), ctypes.byref(self.c_w),
                  ctypes.c_void_p(u_host.data_ptr()), ctypes.c_void_p(out_host.data_ptr()), b, l, _p(ws), ws.numel(), _stream(),
                  1 if overlap else 0)
        return out_host

    def decode(self, u_t, cache, out=None):
        """One token per sequence: u_t (b,d_model); cache advanced in place."""
        b = u_t.shape[0]
        assert u_t.is_contiguous() and u_t.dtype == self.dtype
        lib = capi.load()
        ws = self._ensure_ws(lib.b200_mamba2_mixer_decode_workspace_bytes(ctypes.byref(self.c_cfg), _DT[self.dtype], b))
        if out is None:
            out = torch.empty_like(u_t)
        capi.call("b200_mamba2_mixer_decode", _DT[self.dtype], ctypes.byref(self.c_cfg), ctypes.byref(self.c_w), _p(u_t), _p(out),
                  _p(cache.conv_state), _p(cache.ssm_state), b, _p(ws), ws.numel(), _stream())
        return out

    def capture_decode(self, u_t, cache, out):
        """Records one decode step into a CUDA graph over the fixed buffers `u_t`, `cache` and `out`; `.replay()` of the returned
        graph then advances the cache by one token with a single launch from the host (a decode step is a handful of
        microsecond-scale kernels, so launching them one by one costs as much host time as they take on the device). The cache
        holds the same values after this call as before it."""
        keep = (cache.conv_state.clone(), cache.ssm_state.clone())
        self.decode(u_t, cache, out=out)  # first use: workspace, kernel attributes and tensor maps are set up outside the capture
        cache.conv_state.copy_(keep[0])
        cache.ssm_state.copy_(keep[1])
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.decode(u_t, cache, out=out)
        return graph

    def capture_decode_steps(self, u_steps, cache, out_steps):
        """Records u_steps.shape[0] consecutive decode steps (inputs u_steps[t], outputs out_steps[t], both (steps, b, d_model))
        into ONE CUDA graph: for a run of steps whose inputs are known up front (a benchmark, speculative or teacher-forced
        decoding) the steps then follow each other without a host launch in between, and the first projection of step t+1
        starts (programmatic dependent launch) while the last kernel of step t drains. The cache is left as it was."""
        keep = (cache.conv_state.clone(), cache.ssm_state.clone())
        self.decode(u_steps[0], cache, out=out_steps[0])
        cache.conv_state.copy_(keep[0])
        cache.ssm_state.copy_(keep[1])
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for t in range(u_steps.shape[0]):
                self.decode(u_steps[t], cache, out=out_steps[t])
        return graph


class Mamba2DecoderLayer:
    """The Zamba2 Mamba decoder layer around the mixer: out = hidden + mixer(rms_norm(hidden) * input_norm_weight).
    One C-ABI call per prefill / decode step; the residual is added inside the last projection."""

    def __init__(self, cfg, weights, input_norm_weight, rms_eps=1e-5):
        self.mixer = Mamba2Mixer(cfg, weights)
        self.norm_w, self.rms_eps = input_norm_weight.contiguous(), float(rms_eps)
        self.dtype = self.mixer.dtype

    def prefill(self, hidden, cache=None, initial_states=None, out=None):
        b, l, _ = hidden.shape
        assert hidden.is_contiguous() and hidden.dtype == self.dtype
        m, lib = self.mixer, capi.load()
        ws = m._ensure_ws(lib.b200_mamba2_decoder_prefill_workspace_bytes(ctypes.byref(m.c_cfg), _DT[self.dtype], b, l))
        if out is None:
            out = torch.empty_like(hidden)
        capi.call("b200_mamba2_decoder_prefill", _DT[self.dtype], ctypes.byref(m.c_cfg), ctypes.byref(m.c_w), _p(self.norm_w),
                  self.rms_eps, _p(hidden), _p(out), b, l, _p(initial_states), _p(cache.conv_state) if cache else None,
                  _p(cache.ssm_state) if cache else None, _p(ws), ws.numel(), _stream())
        return out

    def decode(self, hidden_t, cache, out=None):
        b = hidden_t.shape[0]
        assert hidden_t.is_contiguous() and hidden_t.dtype == self.dtype
        m, lib = self.mixer, capi.load()
        ws = m._ensure_ws(lib.b200_mamba2_decoder_decode_workspace_bytes(ctypes.byref(m.c_cfg), _DT[self.dtype], b))
        if out is None:
            out = torch.empty_like(hidden_t)
        capi.call("b200_mamba2_decoder_decode", _DT[self.dtype], ctypes.byref(m.c_cfg), ctypes.byref(m.c_w), _p(self.norm_w),
                  self.rms_eps, _p(hidden_t), _p(out), _p(cache.conv_state), _p(cache.ssm_state), b, _p(ws), ws.numel(), _stream())
        return out


class Mamba2MixerSP:
    """One rank of a sequence-parallel prefill: the rank holds one segment of every sequence. `begin` -> exchange (the caller
    all-gathers the two small tensors it returns) -> `prefix` -> `finish`."""

    def __init__(self, cfg, weights):
        self.cfg, self.w = cfg, weights
        self.c_cfg, self.c_w = make_config(cfg), weights.c_struct()
        self.dtype, self.device = weights.in_proj_weight.dtype, weights.in_proj_weight.device
        self._ws = None
        self._shape = None

    def begin(self, u_seg, u_halo=None, cache=None):
        """u_seg (b, seglen, d_model); u_halo (b, d_conv-1, d_model): the tokens just before the segment (None for the first
        segment). Returns (seg_state (b,H,P,N) fp32, seg_logdecay (b,H) fp32); cache.conv_state receives the segment's last
        conv inputs when a cache is given."""
        b, l, _ = u_seg.shape
        assert u_seg.is_contiguous() and u_seg.dtype == self.dtype and (u_halo is None or u_halo.is_contiguous())
        lib = capi.load()
        nbytes = lib.b200_mamba2_mixer_prefill_sp_workspace_bytes(ctypes.byref(self.c_cfg), _DT[self.dtype], b, l)
        if self._ws is None or self._ws.numel() < nbytes:
            self._ws = _workspace(nbytes, self.device)
        self._shape = (b, l)
        c = self.cfg
        seg_state = torch.empty((b, c["nheads"], c["headdim"], c["d_state"]), dtype=torch.float32, device=self.device)
        seg_logdecay = torch.empty((b, c["nheads"]), dtype=torch.float32, device=self.device)
        capi.call("b200_mamba2_mixer_prefill_sp_begin", _DT[self.dtype], ctypes.byref(self.c_cfg), ctypes.byref(self.c_w), _p(u_seg),
                  _p(u_halo), b, l, _p(seg_state), _p(seg_logdecay), _p(cache.conv_state) if cache else None, _p(self._ws),
                  self._ws.numel(), _stream())
        return seg_state, seg_logdecay

    def prefix(self, seg_states, seg_logdecay, rank):
        """State entering segment `rank` from the gathered per-segment results (R,b,H,P,N) and (R,b,H)."""
        R, b, H, P, N = seg_states.shape
        assert seg_states.is_contiguous() and seg_logdecay.is_contiguous() and seg_states.dtype == torch.float32
        state_in = torch.empty((b, H, P, N), dtype=torch.float32, device=seg_states.device)
        capi.call("b200_ssm_segment_prefix", _p(seg_states), _p(seg_logdecay), int(rank), b, H, P, N, _p(state_in), _stream())
        return state_in

    def finish(self, state_in, out=None, cache=None):
        b, l = self._shape
        if out is None:
            out = torch.empty((b, l, self.cfg["d_model"]), dtype=self.dtype, device=self.device)
        capi.call("b200_mamba2_mixer_prefill_sp_finish", _DT[self.dtype], ctypes.byref(self.c_cfg), ctypes.byref(self.c_w), _p(out), b, l,
                  _p(state_in), _p(cache.ssm_state) if cache else None, _p(self._ws), self._ws.numel(), _stream())
        return out


class Mamba2MixerTP:
    """One rank of the head-sharded (tensor-parallel) prefill mixer. `cfg_local` / `weights` are the rank's local sizes and
    slices (anygpu_b200.synth.tp_local_config / shard_weights_tp). `partial` runs everything up to the rank's out_proj addend;
    the caller sums `partial_out` and `sumsq` over ranks (one all-reduce each) and calls `finish`."""

    def __init__(self, cfg_local, weights, d_inner_global):
        self.cfg, self.w, self.d_inner_global = cfg_local, weights, d_inner_global
        self.c_cfg, self.c_w = make_config(cfg_local), weights.c_struct()
        self.dtype, self.device = weights.in_proj_weight.dtype, weights.in_proj_weight.device
        self._ws = None

    def partial(self, u, partial_out=None, sumsq=None):
        b, l, d_model = u.shape
        assert u.is_contiguous() and u.dtype == self.dtype
        lib = capi.load()
        nbytes = lib.b200_mamba2_mixer_prefill_tp_workspace_bytes(ctypes.byref(self.c_cfg), _DT[self.dtype], b, l)
        if self._ws is None or self._ws.numel() < nbytes:
            self._ws = _workspace(nbytes, self.device)
        if partial_out is None:
            partial_out = torch.empty_like(u)
        if sumsq is None:
            sumsq = torch.empty(b * l, dtype=torch.float32, device=u.device)
        capi.call("b200_mamba2_mixer_prefill_tp_partial", _DT[self.dtype], ctypes.byref(self.c_cfg), ctypes.byref(self.c_w), _p(u),
                  _p(partial_out), _p(sumsq), b, l, None, None, _p(self._ws), self._ws.numel(), _stream())
        return partial_out, sumsq

    def finish(self, out_sum, sumsq_sum):
        rows = sumsq_sum.numel()
        capi.call("b200_mamba2_mixer_tp_finish", _DT[self.dtype], _p(out_sum), _p(sumsq_sum), rows, out_sum.shape[-1],
                  self.d_inner_global, float(self.cfg["eps"]), _stream())
        return out_sum


def tensor_zamba_mamba2_mixer(weights, cache, hidden_states, cfg):
    """Functional form in the argument order of anyGPU's Zamba2 blocks (weights, cache, hidden states, config)."""
    m = Mamba2Mixer(cfg, weights)
    if hidden_states.dim() == 3:
        return m.prefill(hidden_states, cache)
    return m.decode(hidden_states, cache)
