// The device bodies of the fused model kernels (bias + ReLU forward / backward with the
// bias-gradient reduction, 2x2 max pooling forward / backward), compiled for the host
// (-DBAGUA_HOST_EMULATION) and run with one OS thread per CUDA thread on grids of a few blocks,
// compared element for element with the host restatement in model_ops_cpu.cc.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <random>
#include <thread>
#include <vector>

#include "kernels/model_ops.h"
#include "kernels/model_ops_bodies.cuh"

using namespace bagua;
using namespace bagua::model_ops;
using namespace bagua::model_ops::bodies;

namespace {

// 16-byte aligned bf16 storage
struct alignas(16) Vec8 {
  uint16_t h[8];
};
using Buf = std::vector<Vec8>;
uint16_t* raw(Buf& b) { return reinterpret_cast<uint16_t*>(b.data()); }
const uint16_t* raw(const Buf& b) { return reinterpret_cast<const uint16_t*>(b.data()); }

uint16_t to_bf16(float f) {
  uint32_t bits;
  std::memcpy(&bits, &f, 4);
  bits += 0x7fffu + ((bits >> 16) & 1u);
  return (uint16_t)(bits >> 16);
}

// values on a coarse grid (ties), optionally clamped at zero like a ReLU output
void fill(Buf& b, std::mt19937& rng, bool relu) {
  std::normal_distribution<float> n(0.f, 1.f);
  for (auto& v : b)
    for (auto& h : v.h) {
      float x = std::round(n(rng) * 4.f) / 4.f;
      if (relu && x < 0.f) x = 0.f;
      h = to_bf16(x);
    }
}

// Runs fn() as a grid of `blocks` x `threads` CUDA threads.
void launch(int blocks, int threads, const std::function<void()>& fn) {
  std::vector<std::unique_ptr<hostemu::BlockContext>> ctx;
  for (int b = 0; b < blocks; ++b) ctx.push_back(std::make_unique<hostemu::BlockContext>(threads));
  std::vector<std::thread> ts;
  for (int b = 0; b < blocks; ++b)
    for (int t = 0; t < threads; ++t)
      ts.emplace_back([&, b, t] {
        hostemu::bind_thread(ctx[(size_t)b].get(), (unsigned)t, (unsigned)b, (unsigned)blocks);
        fn();
      });
  for (auto& t : ts) t.join();
}

int check_bias_relu(int64_t rows, int C, int blocks, std::mt19937& rng) {
  const int cgroups = C / 8;
  const int64_t nvec = rows * cgroups;
  Buf z((size_t)nvec), bias((size_t)cgroups), want;
  fill(z, rng, false);
  fill(bias, rng, false);
  want = z;
  bias_relu_inplace_bf16_host(raw(want), raw(bias), rows, C);
  launch(blocks, kThreads, [&] {
    bias_relu_body(reinterpret_cast<uint4*>(z.data()), reinterpret_cast<const __nv_bfloat16*>(raw(bias)), nvec, cgroups);
  });
  int bad = std::memcmp(z.data(), want.data(), (size_t)nvec * 16) != 0;

  // backward on the forward's output
  Buf dy((size_t)nvec), dz((size_t)nvec), dz_want((size_t)nvec);
  fill(dy, rng, false);
  std::vector<float> db_want((size_t)C), db((size_t)C, -1.f), partial((size_t)blocks * (size_t)C, -1.f);
  bias_relu_backward_bf16_host(raw(dy), raw(z), raw(dz_want), db_want.data(), rows, C);
  std::vector<std::vector<float>> sacc((size_t)blocks, std::vector<float>((size_t)kThreads * 8));
  launch(blocks, kThreads, [&] {
    bias_relu_backward_body(reinterpret_cast<const uint4*>(dy.data()), reinterpret_cast<const uint4*>(z.data()),
                            reinterpret_cast<uint4*>(dz.data()), partial.data(), rows, cgroups,
                            sacc[hostemu::t_block_idx.x].data());
  });
  launch((C + 127) / 128, 128, [&] { bias_grad_finish_body(partial.data(), db.data(), blocks, C); });
  bad += std::memcmp(dz.data(), dz_want.data(), (size_t)nvec * 16) != 0;
  for (int c = 0; c < C; ++c)
    if (std::fabs(db[(size_t)c] - db_want[(size_t)c]) > 1e-3f * (1.f + std::fabs(db_want[(size_t)c]))) ++bad;
  return bad;
}

int check_maxpool(int64_t N, int64_t H, int64_t W, int C, int blocks, std::mt19937& rng) {
  const int cgroups = C / 8;
  const int64_t nin = N * H * W * cgroups, nout = N * (H / 2) * (W / 2) * cgroups;
  Buf x((size_t)nin), y((size_t)nout), y_want((size_t)nout), dy((size_t)nout), dx((size_t)nin), dx_want((size_t)nin);
  fill(x, rng, true);
  fill(dy, rng, false);
  for (auto& v : dx)
    for (auto& h : v.h) h = 0x7fc0;  // every element must be overwritten
  maxpool2x2_forward_bf16_host(raw(x), raw(y_want), N, H, W, C);
  maxpool2x2_backward_bf16_host(raw(x), raw(dy), raw(dx_want), N, H, W, C);
  launch(blocks, kThreads, [&] {
    maxpool2x2_forward_body(reinterpret_cast<const uint4*>(x.data()), reinterpret_cast<uint4*>(y.data()), nout, W / 2, W,
                            cgroups);
  });
  launch(blocks, kThreads, [&] {
    maxpool2x2_backward_body(reinterpret_cast<const uint4*>(x.data()), reinterpret_cast<const uint4*>(dy.data()),
                             reinterpret_cast<uint4*>(dx.data()), nout, W / 2, W, cgroups);
  });
  return (std::memcmp(y.data(), y_want.data(), (size_t)nout * 16) != 0) +
         (std::memcmp(dx.data(), dx_want.data(), (size_t)nin * 16) != 0);
}

int check_bias_relu_pool(int64_t N, int64_t H, int64_t W, int C, int blocks, std::mt19937& rng) {
  const int cgroups = C / 8;
  const int64_t nin = N * H * W * cgroups, nout = N * (H / 2) * (W / 2) * cgroups;
  Buf y((size_t)nin), p((size_t)nout), bias((size_t)cgroups), y_want, p_want((size_t)nout);
  fill(y, rng, false);
  fill(bias, rng, false);
  y_want = y;
  bias_relu_pool_bf16_host(raw(y_want), raw(p_want), raw(bias), N, H, W, C);
  launch(blocks, kThreads, [&] {
    bias_relu_pool_body(reinterpret_cast<uint4*>(y.data()), reinterpret_cast<uint4*>(p.data()),
                        reinterpret_cast<const __nv_bfloat16*>(raw(bias)), N * (H / 2) * (W / 2), W / 2, W, cgroups);
  });
  int bad = (std::memcmp(y.data(), y_want.data(), (size_t)nin * 16) != 0) +
            (std::memcmp(p.data(), p_want.data(), (size_t)nout * 16) != 0);

  Buf dp((size_t)nout), dz((size_t)nin), dz_want((size_t)nin);
  fill(dp, rng, false);
  for (auto& v : dz)
    for (auto& h : v.h) h = 0x7fc0;  // every element must be overwritten
  std::vector<float> db_want((size_t)C), db((size_t)C, -1.f), partial((size_t)blocks * (size_t)C, -1.f);
  bias_relu_pool_backward_bf16_host(raw(dp), raw(y), raw(dz_want), db_want.data(), N, H, W, C);
  std::vector<std::vector<float>> sacc((size_t)blocks, std::vector<float>((size_t)kThreads * 8));
  launch(blocks, kThreads, [&] {
    bias_relu_pool_backward_body(reinterpret_cast<const uint4*>(dp.data()), reinterpret_cast<const uint4*>(y.data()),
                                 reinterpret_cast<uint4*>(dz.data()), partial.data(), N * (H / 2) * (W / 2), W / 2, W,
                                 cgroups, sacc[hostemu::t_block_idx.x].data());
  });
  launch((C + 127) / 128, 128, [&] { bias_grad_finish_body(partial.data(), db.data(), blocks, C); });
  bad += std::memcmp(dz.data(), dz_want.data(), (size_t)nin * 16) != 0;
  for (int c = 0; c < C; ++c)
    if (std::fabs(db[(size_t)c] - db_want[(size_t)c]) > 1e-3f * (1.f + std::fabs(db_want[(size_t)c]))) ++bad;
  return bad;
}

}  // namespace

int main() {
  std::mt19937 rng(7);
  int failures = 0, cases = 0;
  const struct {
    int64_t rows;
    int C, blocks;
  } br[] = {{1, 8, 1}, {37, 64, 2}, {300, 128, 3}, {1031, 256, 2}, {64, 512, 3}, {5, 2048, 2}, {5000, 16, 3}};
  for (const auto& c : br) {
    if (!bias_relu_supported(c.rows, c.C)) {
      std::fprintf(stderr, "shape [%lld, %d] unexpectedly unsupported\n", (long long)c.rows, c.C);
      ++failures;
      continue;
    }
    const int bad = check_bias_relu(c.rows, c.C, c.blocks, rng);
    if (bad) std::fprintf(stderr, "bias+ReLU [%lld, %d] on %d blocks: %d mismatches\n", (long long)c.rows, c.C, c.blocks, bad);
    failures += bad != 0;
    ++cases;
  }
  const struct {
    int64_t N, H, W;
    int C, blocks;
  } mp[] = {{1, 2, 2, 8, 1}, {2, 6, 10, 64, 2}, {3, 8, 4, 128, 3}, {1, 14, 14, 512, 2}, {5, 4, 6, 24, 3}};
  for (const auto& c : mp) {
    const int bad = check_maxpool(c.N, c.H, c.W, c.C, c.blocks, rng);
    if (bad)
      std::fprintf(stderr, "max-pool [%lld, %lld, %lld, %d] on %d blocks: mismatch\n", (long long)c.N, (long long)c.H,
                   (long long)c.W, c.C, c.blocks);
    failures += bad != 0;
    ++cases;
  }
  const struct {
    int64_t N, H, W;
    int C, blocks;
  } bp[] = {{1, 2, 2, 8, 1}, {2, 6, 10, 64, 2}, {3, 8, 4, 128, 3}, {1, 14, 14, 512, 2}, {4, 4, 6, 16, 3}};
  for (const auto& c : bp) {
    const int bad = check_bias_relu_pool(c.N, c.H, c.W, c.C, c.blocks, rng);
    if (bad)
      std::fprintf(stderr, "bias+ReLU+pool [%lld, %lld, %lld, %d] on %d blocks: %d mismatches\n", (long long)c.N,
                   (long long)c.H, (long long)c.W, c.C, c.blocks, bad);
    failures += bad != 0;
    ++cases;
  }
  // index arithmetic on both sides of the 32-bit limit, against plain 64-bit division
  {
    const int64_t big = (int64_t)1 << 32;
    const int64_t as[] = {0, 1, 255, big - 1, big, big + 5, ((int64_t)1 << 40) + 123, ((int64_t)1 << 46) - 1};
    const int64_t ds[] = {1, 3, 8, 112, ((int64_t)1 << 31), big - 1, big + 1};
    int bad = 0;
    for (int64_t a : as)
      for (int64_t d : ds) {
        int64_t q = -1, r = -1;
        div_mod(a, d, q, r);
        bad += q != a / d || r != a % d;
      }
    for (int64_t p : {(int64_t)0, (int64_t)111, (int64_t)112, big - 1, big, big + 113}) {
      const int64_t Wo = 112, W = 224, cg = 5;
      const int cgroups = 8;
      const PoolIndex i = pool_index(p, cg, Wo, W, cgroups);
      const int64_t wo = p % Wo, row = p / Wo;  // row = n * Ho + ho
      bad += i.x00 != ((2 * row) * W + 2 * wo) * cgroups + cg || i.dw != cgroups || i.dh != W * cgroups;
    }
    if (bad) std::fprintf(stderr, "index arithmetic: %d mismatches\n", bad);
    failures += bad != 0;
    ++cases;
  }
  std::printf("model-op emulation: %d cases, %d failures\n", cases, failures);
  return failures ? 1 : 0;
}
