"""Host-side mirror of the reference's kernel launch contract over the C ABI.

Function names, argument order and meaning follow
Kasamix/redline-llm src/kernels/kernels.cuh (LaunchRmsNorm ... LaunchSiluMul);
tensors are torch CUDA tensors (FP16 data as float16 or as int16/uint16 bit
patterns) used only as device memory. Every call goes to libredline_b200.so;
there is no other implementation behind these names, so a missing library or a
non-zero status raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# REDLINE_B200_LIB points at another build of the same library (e.g. one compiled with other tuning macros)
_LIB_PATH = os.environ.get("REDLINE_B200_LIB") or os.path.join(_HERE, "libredline_b200.so")
_lib = None

ABI_SYMBOLS = (
    "rl_version", "rl_last_error", "rl_kernels_init", "rl_launch_rmsnorm",
    "rl_launch_rmsnorm_residual", "rl_launch_rope_inplace", "rl_launch_kv_scatter",
    "rl_launch_paged_attention_decode", "rl_launch_paged_attention_decode_check",
    "rl_launch_silu_mul", "rl_attention_health", "rl_launch_paged_attention_decode_static",
    "rl_launch_embed_gather", "rl_launch_greedy_argmax", "rl_launch_rope_kv_scatter",
    "rl_attention_set_prologue_overlap", "rl_launch_kv_gather", "rl_launch_prefill_softmax",
    "rl_launch_decode_linear", "rl_decode_linear_health", "rl_decode_linear_set_stages",
    "rl_decode_linear_set_max_splits", "rl_launch_qkv_rope_kv_scatter", "rl_launch_decode_advance",
    "rl_launch_paged_prefill_attention", "rl_prefill_attention_health", "rl_attention_test_wait_expiry", "rl_prefill_attention_set_split_blocks",
    "rl_prefill_attention_run_length",
)


class KernelError(RuntimeError):
    """A launcher returned a non-zero status (mirrors the RuntimeError the reference's
    Python binding raises for component errors, src/api/pybind.cpp:15-20)."""


def lib() -> C.CDLL:
    """Loads the CUDA library; raises if it was never built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise KernelError(f"{_LIB_PATH} is missing: run `python -m redline_llm_b200.build` "
                              "(nvcc, sm_100a); there is no CPU or PyTorch fallback")
        L = C.CDLL(_LIB_PATH)
        vp, i32, i64, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float
        L.rl_version.restype = C.c_char_p
        L.rl_last_error.restype = C.c_char_p
        L.rl_kernels_init.argtypes = [C.c_int]
        L.rl_launch_rmsnorm.argtypes = [vp, vp, vp, i32, i32, f32, vp]
        L.rl_launch_rmsnorm_residual.argtypes = [vp, vp, vp, vp, i32, i32, f32, vp]
        L.rl_launch_rope_inplace.argtypes = [vp, vp, i64, i64, vp, i32, i32, i32, i32, f32, vp]
        L.rl_launch_kv_scatter.argtypes = [vp, vp, vp, i64, i64, vp, i64, vp, i32, i32, i32, vp]
        att = [vp, i64, vp, i64, vp, vp, vp, i32, i32, i32, i32, i32, f32, vp]
        L.rl_launch_paged_attention_decode.argtypes = att
        L.rl_launch_paged_attention_decode_check.argtypes = att
        L.rl_launch_paged_attention_decode_static.argtypes = att
        L.rl_launch_silu_mul.argtypes = [vp, vp, i32, i32, vp]
        L.rl_attention_health.argtypes = [C.POINTER(C.c_int)]
        L.rl_launch_embed_gather.argtypes = [vp, i64, vp, vp, i32, i32, vp]
        L.rl_launch_greedy_argmax.argtypes = [vp, vp, i32, i32, vp]
        L.rl_attention_set_prologue_overlap.argtypes = [C.c_int]
        L.rl_launch_kv_gather.argtypes = [vp, vp, i64, i64, i64, i64, vp, vp, i32, i32, i32, vp]
        L.rl_launch_prefill_softmax.argtypes = [vp, vp, i32, i32, i32, i32, vp]
        L.rl_launch_rope_kv_scatter.argtypes = [vp, vp, vp, i64, i64, i64, vp, vp, i64, vp, i32, i32, i32, i32, f32, vp]
        L.rl_launch_decode_linear.argtypes = [vp, i64, vp, i64, vp, i64, vp, i32, i32, i32, i32, vp]
        L.rl_decode_linear_health.argtypes = [C.POINTER(C.c_int)]
        L.rl_launch_qkv_rope_kv_scatter.argtypes = [vp, i64, vp, i64, vp, i64, vp, i32, i32, vp, vp, i64, vp,
                                                    i32, i32, i32, f32, vp]
        L.rl_decode_linear_set_stages.argtypes = [C.c_int]
        L.rl_launch_decode_advance.argtypes = [vp, vp, vp, vp, vp, i32, vp]
        L.rl_launch_paged_prefill_attention.argtypes = [vp, i64, vp, i64, vp, vp, i32, i32, i32, i32, i32, i32, f32, vp]
        L.rl_prefill_attention_health.argtypes = [C.POINTER(C.c_int)]
        L.rl_attention_test_wait_expiry.argtypes = [C.c_int, C.c_int64]
        L.rl_prefill_attention_set_split_blocks.argtypes = [C.c_int]
        L.rl_prefill_attention_run_length.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_int32)]
        L.rl_decode_linear_set_max_splits.argtypes = [C.c_int]
        for name in ABI_SYMBOLS[2:]:
            getattr(L, name).restype = C.c_int
        _lib = L
    return _lib


def _check(status: int, what: str) -> None:
    if status != 0:
        raise KernelError(f"{what}: status {status}: {lib().rl_last_error().decode()}")


def _ptr(t, offset_elems: int = 0) -> int:
    return t.data_ptr() + 2 * offset_elems if t is not None else 0


def _stream(stream) -> int:
    if stream is None:
        import torch
        return torch.cuda.current_stream().cuda_stream
    return getattr(stream, "cuda_stream", stream)


def version() -> str:
    return lib().rl_version().decode()


def init(device: int = -1) -> None:
    _check(lib().rl_kernels_init(device), "rl_kernels_init")


def launch_rms_norm(out, input, weight, num_tokens, hidden_size, eps, stream=None):
    _check(lib().rl_launch_rmsnorm(_ptr(out), _ptr(input), _ptr(weight), num_tokens, hidden_size,
                                   eps, _stream(stream)), "LaunchRmsNorm")


def launch_rms_norm_residual(out, residual, input, weight, num_tokens, hidden_size, eps, stream=None):
    _check(lib().rl_launch_rmsnorm_residual(_ptr(out), _ptr(residual), _ptr(input), _ptr(weight),
                                            num_tokens, hidden_size, eps, _stream(stream)),
           "LaunchRmsNormResidual")


def launch_rope_inplace(q, k, q_row_stride, k_row_stride, positions, num_tokens, num_q_heads,
                        num_kv_heads, head_dim, rope_theta, stream=None, q_offset=0, k_offset=0):
    """q/k may be the same buffer with element offsets (q = qkv+0, k = qkv+1536)."""
    _check(lib().rl_launch_rope_inplace(_ptr(q, q_offset), _ptr(k, k_offset), q_row_stride,
                                        k_row_stride, positions.data_ptr(), num_tokens,
                                        num_q_heads, num_kv_heads, head_dim, rope_theta,
                                        _stream(stream)), "LaunchRopeInplace")


def launch_kv_scatter(kv_pool_layer, k, v, k_row_stride, v_row_stride, block_tables,
                      block_table_row_stride, positions, num_tokens, num_kv_heads, head_dim,
                      stream=None, k_offset=0, v_offset=0):
    _check(lib().rl_launch_kv_scatter(_ptr(kv_pool_layer), _ptr(k, k_offset), _ptr(v, v_offset),
                                      k_row_stride, v_row_stride, block_tables.data_ptr(),
                                      block_table_row_stride, positions.data_ptr(), num_tokens,
                                      num_kv_heads, head_dim, _stream(stream)), "LaunchKvScatter")


def launch_paged_attention_decode(out, out_row_stride, q, q_row_stride, kv_pool_layer, block_tables,
                                  seq_lens, num_seqs, max_blocks_per_seq, num_q_heads, num_kv_heads,
                                  head_dim, scale, stream=None, check_kernel=False, q_offset=0):
    fn = (lib().rl_launch_paged_attention_decode_check if check_kernel
          else lib().rl_launch_paged_attention_decode)
    _check(fn(_ptr(out), out_row_stride, _ptr(q, q_offset), q_row_stride, _ptr(kv_pool_layer),
              block_tables.data_ptr(), seq_lens.data_ptr(), num_seqs, max_blocks_per_seq,
              num_q_heads, num_kv_heads, head_dim, scale, _stream(stream)),
           "LaunchPagedAttentionDecode")


def launch_paged_attention_decode_static(out, out_row_stride, q, q_row_stride, kv_pool_layer, block_tables,
                                         seq_lens, num_seqs, max_blocks_per_seq, num_q_heads, num_kv_heads,
                                         head_dim, scale, stream=None, q_offset=0):
    """Attention for callers that may not allocate device memory (a sealed memory budget, a host that
    forbids cudaMalloc after start-up): identical results, scratch taken from a ~1.6 MB array built
    into the library. At most 1024 sequences per call; calls overlapping on one GPU race on that array;
    make the first call on a device outside stream capture."""
    _check(lib().rl_launch_paged_attention_decode_static(
        _ptr(out), out_row_stride, _ptr(q, q_offset), q_row_stride, _ptr(kv_pool_layer),
        block_tables.data_ptr(), seq_lens.data_ptr(), num_seqs, max_blocks_per_seq, num_q_heads,
        num_kv_heads, head_dim, scale, _stream(stream)), "LaunchPagedAttentionDecode (static scratch)")


def launch_rope_kv_scatter(qkv, q_row_stride, kv_pool_layer, block_tables, block_table_row_stride, positions,
                           num_tokens, num_q_heads, num_kv_heads, head_dim, rope_theta, stream=None):
    """RoPE on the Q and K views of one fused qkv buffer (Q | K | V per row) and the scatter of the
    rotated K and of V into the paged pool, in one launch; same results as the two separate launchers."""
    qw, kw = num_q_heads * head_dim, num_kv_heads * head_dim
    _check(lib().rl_launch_rope_kv_scatter(_ptr(qkv), _ptr(qkv, qw), _ptr(qkv, qw + kw), q_row_stride,
                                           q_row_stride, q_row_stride, _ptr(kv_pool_layer),
                                           block_tables.data_ptr(), block_table_row_stride,
                                           positions.data_ptr(), num_tokens, num_q_heads, num_kv_heads,
                                           head_dim, rope_theta, _stream(stream)), "rope + kv scatter")


def launch_kv_gather(khat, vhat, khat_head_stride, khat_row_stride, vhat_head_stride, vhat_row_stride,
                     kv_pool_layer, block_table_row, ctx_len, num_kv_heads, head_dim, stream=None):
    _check(lib().rl_launch_kv_gather(_ptr(khat), _ptr(vhat), khat_head_stride, khat_row_stride, vhat_head_stride,
                                     vhat_row_stride, _ptr(kv_pool_layer), block_table_row.data_ptr(), ctx_len,
                                     num_kv_heads, head_dim, _stream(stream)), "LaunchKvGather")


def launch_prefill_softmax(probs, scores, num_q_heads, chunk_len, kv_len, chunk_start, stream=None):
    _check(lib().rl_launch_prefill_softmax(_ptr(probs), scores.data_ptr(), num_q_heads, chunk_len, kv_len,
                                           chunk_start, _stream(stream)), "LaunchPrefillSoftmax")


def launch_embed_gather(out, out_row_stride, embed, input_ids, num_tokens, hidden_size, stream=None):
    _check(lib().rl_launch_embed_gather(_ptr(out), out_row_stride, _ptr(embed), input_ids.data_ptr(),
                                        num_tokens, hidden_size, _stream(stream)), "LaunchEmbedGather")


def launch_greedy_argmax(out_tokens, logits, num_seqs, vocab_size, stream=None):
    _check(lib().rl_launch_greedy_argmax(out_tokens.data_ptr(), _ptr(logits), num_seqs, vocab_size,
                                         _stream(stream)), "LaunchGreedyArgmax")


def launch_paged_prefill_attention(out, out_row_stride, q, q_row_stride, kv_pool_layer, block_table_row,
                                   max_blocks_per_seq, chunk_start, chunk_len, num_q_heads, num_kv_heads, head_dim,
                                   scale, stream=None, q_offset=0):
    """Causal attention of one prompt chunk of one sequence over its paged cache, fused (no gather, no score
    matrix in global memory): replaces the gather -> scores GEMM -> softmax -> P.V GEMM composite."""
    _check(lib().rl_launch_paged_prefill_attention(
        _ptr(out), out_row_stride, _ptr(q, q_offset), q_row_stride, _ptr(kv_pool_layer), block_table_row.data_ptr(),
        max_blocks_per_seq, chunk_start, chunk_len, num_q_heads, num_kv_heads, head_dim, scale, _stream(stream)),
        "paged prefill attention")


def set_prefill_attention_split_blocks(blocks: int) -> None:
    """Longest run of 128-key blocks per CTA in the prefill attention kernel (0 = chosen per launch)."""
    _check(lib().rl_prefill_attention_set_split_blocks(blocks), "rl_prefill_attention_set_split_blocks")


def prefill_attention_run_length(chunk_start: int, chunk_len: int, num_q_heads: int, sm_count: int) -> int:
    """The longest run of 128-key blocks one CTA would take for this chunk on a device of `sm_count` SMs
    (host arithmetic; no device needed)."""
    out = C.c_int32(0)
    _check(lib().rl_prefill_attention_run_length(chunk_start, chunk_len, num_q_heads, sm_count, C.byref(out)),
           "rl_prefill_attention_run_length")
    return int(out.value)


def prefill_attention_health() -> int:
    flag = C.c_int(0)
    _check(lib().rl_prefill_attention_health(C.byref(flag)), "rl_prefill_attention_health")
    return flag.value


def launch_decode_advance(input_ids, positions, seq_lens, sampled_tokens, control, num_rows, stream=None):
    """Next step's inputs from this step's sampled tokens, in place on the device (control = int32[1 + rows]:
    [0] advance on/off, [1 + i] a scripted token for row i or -1)."""
    _check(lib().rl_launch_decode_advance(input_ids.data_ptr(), positions.data_ptr(), seq_lens.data_ptr(),
                                          sampled_tokens.data_ptr(), control.data_ptr(), num_rows,
                                          _stream(stream)), "decode advance")


def set_attention_prologue_overlap(enable: bool) -> None:
    """Overlap the attention kernel's table walk with the previous kernel's tail (programmatic
    dependent launch). seq_lens / block_tables must then not be written by the kernel launched
    immediately before attention."""
    _check(lib().rl_attention_set_prologue_overlap(1 if enable else 0), "rl_attention_set_prologue_overlap")


def attention_test_wait_expiry(drop_first_copy: bool, wait_cycles: int = 0) -> None:
    """Test hook: make one warp's first page copy never start and/or shorten every wait's limit (0 = default)."""
    _check(lib().rl_attention_test_wait_expiry(1 if drop_first_copy else 0, wait_cycles), "rl_attention_test_wait_expiry")


def attention_health() -> int:
    """0 if every page load of the attention kernel arrived since the last query (synchronises)."""
    flag = C.c_int(0)
    _check(lib().rl_attention_health(C.byref(flag)), "rl_attention_health")
    return flag.value


EPILOGUE_BIAS, EPILOGUE_SILU_MUL = 0, 1


def launch_decode_linear(out, x, weight, bias=None, num_tokens=None, epilogue=EPILOGUE_BIAS, stream=None):
    """out[T, N] = x[T, K] . weight[N, K]^T (+ bias) for T <= 64 token rows (row views of 2-D tensors;
    strides are taken from the tensors). With EPILOGUE_SILU_MUL weight is [2N, K] (gate rows, then up rows)
    and out[T, N] = silu(gate) * up."""
    T = x.shape[0] if num_tokens is None else num_tokens
    N = out.shape[1]
    _check(lib().rl_launch_decode_linear(_ptr(out), out.stride(0), _ptr(x), x.stride(0), _ptr(weight),
                                         weight.stride(0), _ptr(bias), T, N, x.shape[1], epilogue,
                                         _stream(stream)), "decode linear")


def launch_qkv_rope_kv_scatter(qkv, x, weight, bias, kv_pool_layer, block_tables, block_table_row_stride, positions,
                               num_tokens, num_q_heads, num_kv_heads, head_dim, rope_theta, stream=None):
    """The QKV projection with RoPE and the KV scatter in its epilogue: one launch for
    launch_decode_linear + launch_rope_inplace + launch_kv_scatter, same bits."""
    _check(lib().rl_launch_qkv_rope_kv_scatter(_ptr(qkv), qkv.stride(0), _ptr(x), x.stride(0), _ptr(weight),
                                               weight.stride(0), _ptr(bias), num_tokens, x.shape[1],
                                               _ptr(kv_pool_layer), block_tables.data_ptr(), block_table_row_stride,
                                               positions.data_ptr(), num_q_heads, num_kv_heads, head_dim, rope_theta,
                                               _stream(stream)), "qkv + rope + kv scatter")


def set_decode_linear_stages(stages: int) -> None:
    _check(lib().rl_decode_linear_set_stages(stages), "rl_decode_linear_set_stages")


def set_decode_linear_max_splits(max_splits: int) -> None:
    _check(lib().rl_decode_linear_set_max_splits(max_splits), "rl_decode_linear_set_max_splits")


def decode_linear_health() -> int:
    """0 if every bounded wait of the decode linear kernel completed since the last query (synchronises)."""
    flag = C.c_int(0)
    _check(lib().rl_decode_linear_health(C.byref(flag)), "rl_decode_linear_health")
    return flag.value


def launch_silu_mul(out, gate_up, num_tokens, intermediate_size, stream=None):
    _check(lib().rl_launch_silu_mul(_ptr(out), _ptr(gate_up), num_tokens, intermediate_size,
                                    _stream(stream)), "LaunchSiluMul")
