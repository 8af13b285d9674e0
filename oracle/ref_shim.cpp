// ref_shim.cpp - C-ABI doorway onto the reference's OWN header-only CPU
// implementation (tests/reference/*.hpp of Kasamix/redline-llm), compiled
// from the headers where they lie in the mounted reference tree; nothing of
// the reference is copied into this repository. The Makefile passes
// -I<reference>/tests. Output goes to oracle/_ref/ only.
//
// TEST INFRASTRUCTURE: used to pin oracle/redline_oracle.c and, in the
// benchmark's reference leg, as the timed CPU implementation. Never linked
// into the shipped library.
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "reference/attention_ref.hpp"
#include "reference/elementwise_ref.hpp"
#include "reference/fp16_ref.hpp"
#include "reference/pool_ref.hpp"
#include "reference/rmsnorm_ref.hpp"
#include "reference/rope_ref.hpp"

namespace ref = redline::reference;
using u16 = std::uint16_t;

namespace {
std::vector<u16> Vec(const u16* p, std::size_t n) { return std::vector<u16>(p, p + n); }

// Runs fn(begin, end) over [0, n) on `threads` std::threads (row-parallel
// wrapper around the single-threaded reference functions).
template <typename Fn> void ParallelRows(int n, int threads, Fn fn) {
  if (threads <= 1 || n <= 1) {
    fn(0, n);
    return;
  }
  if (threads > n) threads = n;
  std::vector<std::thread> pool;
  for (int t = 0; t < threads; ++t) {
    const int b = static_cast<int>(static_cast<long long>(n) * t / threads);
    const int e = static_cast<int>(static_cast<long long>(n) * (t + 1) / threads);
    pool.emplace_back([=] { fn(b, e); });
  }
  for (auto& th : pool) th.join();
}
} // namespace

extern "C" {

double rlr_half_to_double(u16 h) { return ref::HalfBitsToDouble(h); }
u16 rlr_quantize(double x) { return ref::QuantizeDoubleToHalfBits(x); }
u16 rlr_half_add(u16 a, u16 b) { return ref::HalfAddRn(a, b); }
double rlr_rel_distance_to_boundary(double v) { return ref::RelDistanceToHalfBoundary(v); }

std::uint64_t rlr_fill_uniform_half(std::uint64_t seed, u16* out, std::int64_t n, double lo,
                                    double hi) {
  // The reference's stream object hides its state; replay from the seed.
  ref::SplitMix64 rng(seed);
  for (std::int64_t i = 0; i < n; ++i) out[i] = rng.NextHalfBitsUniform(lo, hi);
  return 0;
}

void rlr_rmsnorm(u16* out, const u16* in, const u16* w, std::int32_t rows, std::int32_t hidden,
                 float eps, int threads) {
  const auto wv = Vec(w, hidden);
  ParallelRows(rows, threads, [&](int b, int e) {
    const auto r = ref::RmsNormReference(Vec(in + std::size_t(b) * hidden, std::size_t(e - b) * hidden),
                                         wv, e - b, hidden, eps);
    std::memcpy(out + std::size_t(b) * hidden, r.data(), r.size() * 2);
  });
}

void rlr_rmsnorm_residual(u16* out, u16* residual, const u16* in, const u16* w, std::int32_t rows,
                          std::int32_t hidden, float eps, double* inv_rms, std::uint8_t* excluded,
                          double rel_floor, int threads) {
  const auto wv = Vec(w, hidden);
  ParallelRows(rows, threads, [&](int b, int e) {
    const std::size_t off = std::size_t(b) * hidden, n = std::size_t(e - b) * hidden;
    const auto r = ref::ComputeFusedRmsNormReference(Vec(residual + off, n), Vec(in + off, n), wv,
                                                     e - b, hidden, eps, rel_floor);
    std::memcpy(out + off, r.out_bits.data(), n * 2);
    std::memcpy(residual + off, r.residual_bits.data(), n * 2);
    if (inv_rms) std::memcpy(inv_rms + b, r.inv_rms.data(), std::size_t(e - b) * sizeof(double));
    if (excluded) std::memcpy(excluded + off, r.excluded.data(), n);
  });
}

void rlr_rmsnorm_residual_mutant_unrounded(u16* out, const u16* residual, const u16* in,
                                           const u16* w, std::int32_t rows, std::int32_t hidden,
                                           float eps) {
  const std::size_t n = std::size_t(rows) * hidden;
  const auto r = ref::FusedRmsNormMutantUnroundedSum(Vec(residual, n), Vec(in, n), Vec(w, hidden),
                                                     rows, hidden, eps);
  std::memcpy(out, r.data(), n * 2);
}

void rlr_rmsnorm_residual_mutant_single_round(u16* out, const u16* residual, const u16* in,
                                              const u16* w, std::int32_t rows, std::int32_t hidden,
                                              float eps) {
  const std::size_t n = std::size_t(rows) * hidden;
  const auto r = ref::FusedRmsNormMutantSingleRounding(Vec(residual, n), Vec(in, n),
                                                       Vec(w, hidden), rows, hidden, eps);
  std::memcpy(out, r.data(), n * 2);
}

void rlr_build_rmsnorm_boundary_fixture(std::uint64_t seed, u16* residual, u16* input, u16* weight,
                                        std::uint8_t* is_boundary) {
  const auto fx = ref::BuildRmsNormBoundaryFixture(seed);
  std::memcpy(residual, fx.residual.data(), fx.residual.size() * 2);
  std::memcpy(input, fx.input.data(), fx.input.size() * 2);
  std::memcpy(weight, fx.weight.data(), fx.weight.size() * 2);
  if (is_boundary) std::memcpy(is_boundary, fx.is_boundary.data(), fx.is_boundary.size());
}

// Dense rows only (the reference function takes a packed buffer).
void rlr_rope(u16* heads, const std::int32_t* positions, std::int32_t num_tokens,
              std::int32_t num_heads, std::int32_t head_dim, double theta, int threads) {
  const std::size_t w = std::size_t(num_heads) * head_dim;
  ParallelRows(num_tokens, threads, [&](int b, int e) {
    auto v = Vec(heads + b * w, std::size_t(e - b) * w);
    const std::vector<std::int32_t> pos(positions + b, positions + e);
    ref::RopeReferenceInplace(v, pos, e - b, num_heads, head_dim, theta);
    std::memcpy(heads + b * w, v.data(), v.size() * 2);
  });
}

void rlr_kv_scatter(u16* pool, std::int64_t pool_elems, const u16* k, const u16* v,
                    std::int64_t k_row_stride, std::int64_t v_row_stride,
                    const std::int32_t* tables, std::int64_t table_row_stride,
                    const std::int32_t* positions, std::int32_t num_tokens, std::int32_t kv_heads,
                    std::int32_t head_dim) {
  std::vector<u16> p(pool, pool + pool_elems);
  ref::ScatterReference(p, k, v, k_row_stride, v_row_stride, tables, table_row_stride, positions,
                        num_tokens, kv_heads, head_dim);
  std::memcpy(pool, p.data(), std::size_t(pool_elems) * 2);
}

// Rows with seq_len <= 0 come back as +0 bits (the reference function's own
// convention).
void rlr_paged_attention(u16* out, const u16* q, const u16* pool, std::int64_t pool_elems,
                         const std::int32_t* tables, const std::int32_t* seq_lens,
                         std::int32_t num_seqs, std::int32_t max_blocks_per_seq,
                         std::int32_t q_heads, std::int32_t kv_heads, std::int32_t head_dim,
                         double scale, int threads) {
  const std::vector<u16> pv(pool, pool + pool_elems);
  const std::size_t w = std::size_t(q_heads) * head_dim;
  ParallelRows(num_seqs, threads, [&](int b, int e) {
    const std::vector<std::int32_t> tb(tables + std::size_t(b) * max_blocks_per_seq,
                                       tables + std::size_t(e) * max_blocks_per_seq);
    const std::vector<std::int32_t> sl(seq_lens + b, seq_lens + e);
    const auto r = ref::PagedAttentionDecodeReference(Vec(q + b * w, std::size_t(e - b) * w), pv, tb,
                                                      sl, e - b, max_blocks_per_seq, q_heads,
                                                      kv_heads, head_dim, scale);
    std::memcpy(out + b * w, r.data(), r.size() * 2);
  });
}

void rlr_silu_mul(u16* out, const u16* gate_up, std::int32_t rows, std::int32_t inter,
                  int threads) {
  ParallelRows(rows, threads, [&](int b, int e) {
    const auto r = ref::SiluMulReference(
        Vec(gate_up + std::size_t(b) * 2 * inter, std::size_t(e - b) * 2 * inter), e - b, inter);
    std::memcpy(out + std::size_t(b) * inter, r.data(), r.size() * 2);
  });
}

void rlr_argmax(std::int32_t* out, const u16* logits, std::int32_t rows, std::int32_t vocab) {
  const auto r = ref::ArgmaxReference(Vec(logits, std::size_t(rows) * vocab), rows, vocab);
  std::memcpy(out, r.data(), r.size() * sizeof(std::int32_t));
}

void rlr_kv_gather(u16* khat, u16* vhat, std::int64_t khat_head_stride, std::int64_t khat_row_stride,
                   std::int64_t vhat_head_stride, std::int64_t vhat_row_stride, const u16* pool,
                   std::int64_t pool_elems, const std::int32_t* table_row, std::int32_t ctx_len,
                   std::int32_t kv_heads, std::int32_t head_dim) {
  const std::vector<u16> p(pool, pool + pool_elems);
  ref::GatherReference(khat, vhat, khat_head_stride, khat_row_stride, vhat_head_stride, vhat_row_stride, p,
                       table_row, ctx_len, kv_heads, head_dim);
}

void rlr_prefill_softmax(u16* probs, const float* scores, std::int32_t heads, std::int32_t chunk_len,
                         std::int32_t kv_len, std::int32_t chunk_start) {
  const std::size_t n = std::size_t(heads) * chunk_len * kv_len;
  const auto r = ref::PrefillSoftmaxReference(std::vector<float>(scores, scores + n), heads, chunk_len, kv_len,
                                              chunk_start);
  std::memcpy(probs, r.data(), n * 2);
}

int rlr_hardware_threads() { return static_cast<int>(std::thread::hardware_concurrency()); }

} // extern "C"
