// A C++ caller of the drop-in launch header: the call sites look exactly like the
// reference's own (src/core/model_executor.cpp:908-949, tests/test_kernels.cu), namespace
// redline::kernels, half* device pointers, cudaStream_t last. Checks, on a GPU:
//   scatter  - bit-exact against a host mirror of the pool (p >> 4, p & 15 slot math);
//   attention- primary launcher against the per-query-head cross-check launcher (<= 2e-3);
//   silu_mul - in place over the gate half, up half untouched, against host float math (<= 1 FP16 step);
//   fused norm - residual write-back equals a native half add.
// Prints one line per check and exits non-zero on the first failure.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "kernels.cuh"

namespace rk = redline::kernels;

static uint64_t g_state = 0xB200C0DEull;
static double Uniform() {
  g_state += 0x9E3779B97F4A7C15ull;
  uint64_t z = g_state;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return static_cast<double>(z >> 11) * 0x1.0p-53;
}
static std::vector<half> RandomHalves(size_t n, double lo, double hi) {
  std::vector<half> v(n);
  for (auto& x : v) x = __float2half_rn(static_cast<float>(lo + Uniform() * (hi - lo)));
  return v;
}
template <typename T> static T* Upload(const std::vector<T>& v) {
  T* d = nullptr;
  cudaMalloc(&d, v.size() * sizeof(T));
  cudaMemcpy(d, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice);
  return d;
}
template <typename T> static std::vector<T> Download(const T* d, size_t n) {
  std::vector<T> v(n);
  cudaMemcpy(v.data(), d, n * sizeof(T), cudaMemcpyDeviceToHost);
  return v;
}
static uint16_t Bits(half h) { return *reinterpret_cast<uint16_t*>(&h); }
static void Require(bool ok, const char* what) {
  std::printf("%s: %s\n", what, ok ? "ok" : "FAILED");
  if (!ok) std::exit(1);
}

int main() {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
    std::printf("no CUDA device\n");
    return 77;
  }
  cudaStream_t stream;
  cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
  constexpr int kQ = 12, kKv = 2, kD = 128, kQkv = 2048, kBlocks = 96, kSeqs = 5, kMbps = 20;
  const int lens[kSeqs] = {257, 0, 64, 17, 300};

  // ---- block tables: distinct real blocks, dummy-padded
  std::vector<int32_t> tables(kSeqs * kMbps, 0), seq_lens(lens, lens + kSeqs);
  int next = 1;
  for (int s = 0; s < kSeqs; ++s)
    for (int b = 0; b < (lens[s] + 15) / 16; ++b) tables[s * kMbps + b] = next++;
  const size_t pool_elems = static_cast<size_t>(kBlocks) * 2 * kKv * 16 * kD;
  std::vector<half> pool(pool_elems, __ushort_as_half(0x7E00));  // NaN-poisoned
  half* d_pool = Upload(pool);
  int32_t* d_tables = Upload(tables);

  // ---- scatter every live position of every sequence, one qkv-strided batch per position index
  std::vector<half> mirror = pool;
  for (int p = 0; p < 300; ++p) {
    std::vector<int32_t> pos(kSeqs, 0), rows;
    std::vector<half> qkv = RandomHalves(static_cast<size_t>(kSeqs) * kQkv, -1.0, 1.0);
    std::vector<int32_t> tab_rows;
    int live = 0;
    std::vector<half> packed;
    std::vector<int32_t> packed_pos, packed_tab;
    for (int s = 0; s < kSeqs; ++s) {
      if (p >= lens[s]) continue;
      packed.insert(packed.end(), qkv.begin() + s * kQkv, qkv.begin() + (s + 1) * kQkv);
      packed_pos.push_back(p);
      packed_tab.insert(packed_tab.end(), tables.begin() + s * kMbps, tables.begin() + (s + 1) * kMbps);
      for (int h = 0; h < kKv; ++h)
        for (int d = 0; d < kD; ++d) {
          const int block = tables[s * kMbps + (p >> 4)], slot = p & 15;
          mirror[((((size_t)block * 2 + 0) * kKv + h) * 16 + slot) * kD + d] = qkv[s * kQkv + 1536 + h * kD + d];
          mirror[((((size_t)block * 2 + 1) * kKv + h) * 16 + slot) * kD + d] = qkv[s * kQkv + 1792 + h * kD + d];
        }
      ++live;
    }
    if (!live) continue;
    half* d_qkv = Upload(packed);
    int32_t* d_pos = Upload(packed_pos);
    int32_t* d_tab = Upload(packed_tab);
    rk::LaunchKvScatter(d_pool, d_qkv + 1536, d_qkv + 1792, kQkv, kQkv, d_tab, kMbps, d_pos, live, kKv, kD, stream);
    cudaStreamSynchronize(stream);
    cudaFree(d_qkv);
    cudaFree(d_pos);
    cudaFree(d_tab);
  }
  {
    const std::vector<half> got = Download(d_pool, pool_elems);
    bool same = true;
    for (size_t i = 0; i < pool_elems && same; ++i) same = Bits(got[i]) == Bits(mirror[i]);
    Require(same, "LaunchKvScatter bit-exact against the host mirror (NaN-poisoned pool)");
  }

  // ---- attention: primary vs the cross-check launcher, qkv-strided q, padded row untouched
  std::vector<half> q = RandomHalves(static_cast<size_t>(kSeqs) * kQkv, -1.0, 1.0);
  half* d_q = Upload(q);
  int32_t* d_lens = Upload(seq_lens);
  std::vector<half> sentinel(static_cast<size_t>(kSeqs) * kQ * kD, __ushort_as_half(0x1234));
  half* d_out_a = Upload(sentinel);
  half* d_out_b = Upload(sentinel);
  const float scale = 0.088388347648318447f;
  rk::LaunchPagedAttentionDecode(d_out_a, kQ * kD, d_q, kQkv, d_pool, d_tables, d_lens, kSeqs, kMbps, kQ, kKv, kD, scale, stream);
  rk::LaunchPagedAttentionDecodeOracle(d_out_b, kQ * kD, d_q, kQkv, d_pool, d_tables, d_lens, kSeqs, kMbps, kQ, kKv, kD, scale, stream);
  Require(cudaStreamSynchronize(stream) == cudaSuccess, "attention launches complete");
  {
    const auto a = Download(d_out_a, sentinel.size()), b = Download(d_out_b, sentinel.size());
    double worst = 0.0;
    bool padded_untouched = true, finite = true;
    for (int s = 0; s < kSeqs; ++s)
      for (int c = 0; c < kQ * kD; ++c) {
        const size_t i = static_cast<size_t>(s) * kQ * kD + c;
        if (lens[s] <= 0) {
          padded_untouched = padded_untouched && Bits(a[i]) == 0x1234;
        } else {
          const double x = __half2float(a[i]), y = __half2float(b[i]);
          finite = finite && std::isfinite(x);
          worst = std::fmax(worst, std::fabs(x - y));
        }
      }
    Require(padded_untouched, "LaunchPagedAttentionDecode leaves the seq_len 0 row unwritten");
    Require(finite && worst <= 2e-3, "LaunchPagedAttentionDecode matches the cross-check launcher (<= 2e-3)");
  }

  // ---- silu_mul in place over the gate half
  constexpr int kT = 9, kI = 8960;
  std::vector<half> gu = RandomHalves(static_cast<size_t>(kT) * 2 * kI, -3.0, 3.0);
  half* d_gu = Upload(gu);
  rk::LaunchSiluMul(d_gu, d_gu, kT, kI, stream);
  cudaStreamSynchronize(stream);
  {
    const auto got = Download(d_gu, gu.size());
    bool ok = true, up_same = true;
    for (int t = 0; t < kT; ++t)
      for (int c = 0; c < kI; ++c) {
        const float g = __half2float(gu[(size_t)t * 2 * kI + c]), u = __half2float(gu[(size_t)t * 2 * kI + kI + c]);
        const half want = __float2half_rn(g / (1.0f + std::exp(-g)) * u);
        const int d = std::abs(static_cast<int>(Bits(got[(size_t)t * 2 * kI + c]) & 0x7FFF) - static_cast<int>(Bits(want) & 0x7FFF));
        ok = ok && d <= 1;
        up_same = up_same && Bits(got[(size_t)t * 2 * kI + kI + c]) == Bits(gu[(size_t)t * 2 * kI + kI + c]);
      }
    Require(ok, "LaunchSiluMul in place within one FP16 step of host float math");
    Require(up_same, "LaunchSiluMul leaves the up half untouched");
  }

  // ---- fused residual-add + RMSNorm: write-back is the native half add
  constexpr int kH = 1536;
  std::vector<half> x = RandomHalves(static_cast<size_t>(kT) * kH, -1.0, 1.0), r = RandomHalves(static_cast<size_t>(kT) * kH, -1.0, 1.0);
  std::vector<half> w = RandomHalves(kH, 0.5, 1.5);
  half *d_x = Upload(x), *d_r = Upload(r), *d_w = Upload(w), *d_n = Upload(x);
  rk::LaunchRmsNormResidual(d_n, d_r, d_x, d_w, kT, kH, 1e-6f, stream);
  cudaStreamSynchronize(stream);
  {
    const auto res = Download(d_r, r.size()), out = Download(d_n, x.size());
    bool ok = true;
    double worst = 0.0;
    for (int t = 0; t < kT; ++t) {
      double ss = 0.0;
      for (int c = 0; c < kH; ++c) {
        const half h = __float2half_rn(__half2float(r[(size_t)t * kH + c]) + __half2float(x[(size_t)t * kH + c]));
        ok = ok && Bits(h) == Bits(res[(size_t)t * kH + c]);
        ss += static_cast<double>(__half2float(h)) * __half2float(h);
      }
      const double inv = 1.0 / std::sqrt(ss / kH + 1e-6);
      for (int c = 0; c < kH; ++c) {
        const double want = __half2float(__float2half_rn(static_cast<float>(__half2float(res[(size_t)t * kH + c]) * inv))) *
                            static_cast<double>(__half2float(w[c]));
        worst = std::fmax(worst, std::fabs(want - __half2float(out[(size_t)t * kH + c])));
      }
    }
    Require(ok, "LaunchRmsNormResidual writes back fp16(residual + input) exactly");
    Require(worst <= 4e-3, "LaunchRmsNormResidual output within FP16 rounding of the FP64 result");
  }
  // ---- decode-sized linear layer (beyond the reference header): product against a host double sum, and the
  // gated epilogue against the product followed by LaunchSiluMul
  {
    constexpr int kLinT = 9, kLinK = 256, kLinI = 192;
    std::vector<half> lx = RandomHalves(static_cast<size_t>(kLinT) * kLinK, -1.0, 1.0);
    std::vector<half> lw = RandomHalves(static_cast<size_t>(2 * kLinI) * kLinK, -0.0625, 0.0625);
    half *d_lx = Upload(lx), *d_lw = Upload(lw);
    half *d_prod = nullptr, *d_act = nullptr, *d_two = nullptr;
    cudaMalloc(&d_prod, sizeof(half) * kLinT * 2 * kLinI);
    cudaMalloc(&d_act, sizeof(half) * kLinT * kLinI);
    cudaMalloc(&d_two, sizeof(half) * kLinT * kLinI);
    rl_decode_linear_set_max_splits(1);  // the gated product is never split along K: compare like with like
    rk::LaunchDecodeLinear(d_prod, 2 * kLinI, d_lx, kLinK, d_lw, kLinK, nullptr, kLinT, 2 * kLinI, kLinK, false, stream);
    rl_decode_linear_set_max_splits(8);
    rk::LaunchDecodeLinear(d_act, kLinI, d_lx, kLinK, d_lw, kLinK, nullptr, kLinT, kLinI, kLinK, true, stream);
    rk::LaunchSiluMul(d_two, d_prod, kLinT, kLinI, stream);
    cudaStreamSynchronize(stream);
    const auto prod = Download(d_prod, static_cast<size_t>(kLinT) * 2 * kLinI);
    const auto act = Download(d_act, static_cast<size_t>(kLinT) * kLinI), two = Download(d_two, static_cast<size_t>(kLinT) * kLinI);
    double worst = 0.0;
    for (int t = 0; t < kLinT; ++t)
      for (int n = 0; n < 2 * kLinI; ++n) {
        double sum = 0.0;
        for (int k = 0; k < kLinK; ++k) sum += static_cast<double>(__half2float(lx[(size_t)t * kLinK + k])) * __half2float(lw[(size_t)n * kLinK + k]);
        worst = std::fmax(worst, std::fabs(sum - __half2float(prod[(size_t)t * 2 * kLinI + n])));
      }
    bool same = true;
    for (size_t i = 0; i < act.size(); ++i) same = same && Bits(act[i]) == Bits(two[i]);
    Require(worst <= 1.5e-3, "LaunchDecodeLinear within FP16 rounding of the host double product");
    Require(same, "LaunchDecodeLinear with the gated epilogue equals product + LaunchSiluMul bit for bit");
  }
  Require(cudaGetLastError() == cudaSuccess, "no CUDA error left behind");
  std::printf("all checks passed\n");
  return 0;
}
