"""ctypes doorway onto the reference's OWN CUDA kernels (TEST INFRASTRUCTURE).

`oracle/_ref/libredline_refkernels.so` is the reference's src/kernels/*.cu compiled for sm_100a where
they lie (oracle/Makefile, target `gpuref`) behind the C ABI of oracle/ref_kernels_shim.cu. This
module gives it the method names and argument lists of `redline_llm_b200.kernels`, so that a test or
the benchmark can run either library on the same device buffers - and can hand this module to the
decode engine's executor in place of the product's kernel module to drive a whole model through the
reference's kernels. Only tests/, the smoke check and the benchmark's comparator columns import it;
the shipped path never does. `available()` is False where the library was never built.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libredline_refkernels.so")
HOST_B200_DIR = os.path.join(_HERE, "_ref", "host_b200")   # the reference's C++ host over this library's kernels
HOST_REF_DIR = os.path.join(_HERE, "_ref", "host_ref")     # the reference's C++ host over its own kernels
_lib = None

SYMBOLS = ("refk_launch_embed_gather", "refk_launch_rmsnorm", "refk_launch_rmsnorm_residual",
           "refk_launch_rope_inplace", "refk_launch_kv_scatter", "refk_launch_kv_gather",
           "refk_launch_paged_attention_decode", "refk_launch_paged_attention_decode_check",
           "refk_launch_prefill_softmax", "refk_launch_silu_mul", "refk_launch_greedy_argmax")


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not available():
            raise RuntimeError(f"{LIB_PATH} was never built (make -C oracle gpuref, where the reference tree is mounted)")
        L = C.CDLL(LIB_PATH)
        vp, i32, i64, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float
        L.refk_launch_rmsnorm.argtypes = [vp, vp, vp, i32, i32, f32, vp]
        L.refk_launch_rmsnorm_residual.argtypes = [vp, vp, vp, vp, i32, i32, f32, vp]
        L.refk_launch_rope_inplace.argtypes = [vp, vp, i64, i64, vp, i32, i32, i32, i32, f32, vp]
        L.refk_launch_kv_scatter.argtypes = [vp, vp, vp, i64, i64, vp, i64, vp, i32, i32, i32, vp]
        att = [vp, i64, vp, i64, vp, vp, vp, i32, i32, i32, i32, i32, f32, vp]
        L.refk_launch_paged_attention_decode.argtypes = att
        L.refk_launch_paged_attention_decode_check.argtypes = att
        L.refk_launch_silu_mul.argtypes = [vp, vp, i32, i32, vp]
        L.refk_launch_embed_gather.argtypes = [vp, i64, vp, vp, i32, i32, vp]
        L.refk_launch_greedy_argmax.argtypes = [vp, vp, i32, i32, vp]
        L.refk_launch_kv_gather.argtypes = [vp, vp, i64, i64, i64, i64, vp, vp, i32, i32, i32, vp]
        L.refk_launch_prefill_softmax.argtypes = [vp, vp, i32, i32, i32, i32, vp]
        for name in SYMBOLS:
            getattr(L, name).restype = C.c_int
        _lib = L
    return _lib


def _check(status: int, what: str) -> None:
    if status != 0:
        raise RuntimeError(f"reference kernel {what}: cudaError {status}")


def _ptr(t, offset_elems: int = 0) -> int:
    return t.data_ptr() + 2 * offset_elems if t is not None else 0


def _stream(stream) -> int:
    if stream is None:
        import torch
        return torch.cuda.current_stream().cuda_stream
    return getattr(stream, "cuda_stream", stream)


def init(device: int = -1) -> None:   # the reference's kernels keep no state that needs an explicit set-up
    lib()


def launch_rms_norm(out, input, weight, num_tokens, hidden_size, eps, stream=None):
    _check(lib().refk_launch_rmsnorm(_ptr(out), _ptr(input), _ptr(weight), num_tokens, hidden_size, eps,
                                     _stream(stream)), "LaunchRmsNorm")


def launch_rms_norm_residual(out, residual, input, weight, num_tokens, hidden_size, eps, stream=None):
    _check(lib().refk_launch_rmsnorm_residual(_ptr(out), _ptr(residual), _ptr(input), _ptr(weight), num_tokens,
                                              hidden_size, eps, _stream(stream)), "LaunchRmsNormResidual")


def launch_rope_inplace(q, k, q_row_stride, k_row_stride, positions, num_tokens, num_q_heads, num_kv_heads,
                        head_dim, rope_theta, stream=None, q_offset=0, k_offset=0):
    _check(lib().refk_launch_rope_inplace(_ptr(q, q_offset), _ptr(k, k_offset), q_row_stride, k_row_stride,
                                          positions.data_ptr(), num_tokens, num_q_heads, num_kv_heads, head_dim,
                                          rope_theta, _stream(stream)), "LaunchRopeInplace")


def launch_kv_scatter(kv_pool_layer, k, v, k_row_stride, v_row_stride, block_tables, block_table_row_stride,
                      positions, num_tokens, num_kv_heads, head_dim, stream=None, k_offset=0, v_offset=0):
    _check(lib().refk_launch_kv_scatter(_ptr(kv_pool_layer), _ptr(k, k_offset), _ptr(v, v_offset), k_row_stride,
                                        v_row_stride, block_tables.data_ptr(), block_table_row_stride,
                                        positions.data_ptr(), num_tokens, num_kv_heads, head_dim,
                                        _stream(stream)), "LaunchKvScatter")


def launch_paged_attention_decode(out, out_row_stride, q, q_row_stride, kv_pool_layer, block_tables, seq_lens,
                                  num_seqs, max_blocks_per_seq, num_q_heads, num_kv_heads, head_dim, scale,
                                  stream=None, check_kernel=False, q_offset=0):
    fn = lib().refk_launch_paged_attention_decode_check if check_kernel else lib().refk_launch_paged_attention_decode
    _check(fn(_ptr(out), out_row_stride, _ptr(q, q_offset), q_row_stride, _ptr(kv_pool_layer),
              block_tables.data_ptr(), seq_lens.data_ptr(), num_seqs, max_blocks_per_seq, num_q_heads,
              num_kv_heads, head_dim, scale, _stream(stream)), "LaunchPagedAttentionDecode")


def launch_kv_gather(khat, vhat, khat_head_stride, khat_row_stride, vhat_head_stride, vhat_row_stride,
                     kv_pool_layer, block_table_row, ctx_len, num_kv_heads, head_dim, stream=None):
    _check(lib().refk_launch_kv_gather(_ptr(khat), _ptr(vhat), khat_head_stride, khat_row_stride, vhat_head_stride,
                                       vhat_row_stride, _ptr(kv_pool_layer), block_table_row.data_ptr(), ctx_len,
                                       num_kv_heads, head_dim, _stream(stream)), "LaunchKvGather")


def launch_prefill_softmax(probs, scores, num_q_heads, chunk_len, kv_len, chunk_start, stream=None):
    _check(lib().refk_launch_prefill_softmax(_ptr(probs), scores.data_ptr(), num_q_heads, chunk_len, kv_len,
                                             chunk_start, _stream(stream)), "LaunchPrefillSoftmax")


def launch_embed_gather(out, out_row_stride, embed, input_ids, num_tokens, hidden_size, stream=None):
    _check(lib().refk_launch_embed_gather(_ptr(out), out_row_stride, _ptr(embed), input_ids.data_ptr(), num_tokens,
                                          hidden_size, _stream(stream)), "LaunchEmbedGather")


def launch_greedy_argmax(out_tokens, logits, num_seqs, vocab_size, stream=None):
    _check(lib().refk_launch_greedy_argmax(out_tokens.data_ptr(), _ptr(logits), num_seqs, vocab_size,
                                           _stream(stream)), "LaunchGreedyArgmax")


def launch_silu_mul(out, gate_up, num_tokens, intermediate_size, stream=None):
    _check(lib().refk_launch_silu_mul(_ptr(out), _ptr(gate_up), num_tokens, intermediate_size, _stream(stream)),
           "LaunchSiluMul")
