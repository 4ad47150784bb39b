// GPU test of the C++ Backend mirror (include/tpb200.hpp), written the way the
// reference's device tests are (src/gpu/cuda/kernels.zig:2557-2701,
// src/gpu/cuda/backend.zig:3727-3792): host weights and activations in, one op
// sequence through the Backend, results compared with the CPU checker.
// The checker (oracle/) is test infrastructure: it is linked here and nowhere else.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <vector>

#include "tpb200.hpp"
extern "C" {
#include "tpb_oracle.h"
}

static int failures = 0;
#define EXPECT(cond, ...)                       \
    do {                                        \
        if (!(cond)) {                          \
            std::printf("FAIL %s:%d: ", __FILE__, __LINE__); \
            std::printf(__VA_ARGS__);           \
            std::printf("\n");                  \
            failures++;                         \
        }                                       \
    } while (0)

static void convrot_linear(tpb::Backend &be, int bits, size_t m, size_t n, size_t k, unsigned seed) {
    std::mt19937 rng(seed);
    std::normal_distribution<float> nd(0.f, 1.f);
    std::uniform_real_distribution<float> us(1e-3f, 1e-2f);
    std::vector<float> x(m * k), ws(n);
    for (auto &v : x) v = nd(rng);
    for (size_t i = 0; i < m; i++) x[i * k + 7] *= 30.f;  // an outlier channel, what the rotation is for
    for (auto &v : ws) v = us(rng);
    std::vector<int8_t> w(n * k);
    const int lo = bits == 4 ? -8 : -127, hi = bits == 4 ? 7 : 127;
    std::uniform_int_distribution<int> wi(lo, hi);
    for (auto &v : w) v = (int8_t)wi(rng);
    std::vector<uint8_t> packed(n * k / 2);
    if (bits == 4) tpo_pack_i4(w.data(), n * k, packed.data());

    // checker: integer replica (prep -> int32 GEMM -> dequant)
    std::vector<int8_t> q(m * k);
    std::vector<float> as(m);
    tpo_convrot_prep(x.data(), m, k, bits, q.data(), as.data(), nullptr);
    std::vector<int32_t> acc(m * n);
    tpo_igemm_s32(q.data(), w.data(), m, n, k, acc.data());
    std::vector<double> sim(m * n);
    tpo_dequant_sim(acc.data(), as.data(), ws.data(), m, n, sim.data());

    tpb::DeviceBuffer xd = be.tensorCreate(m * k * 4), yd = be.tensorCreate(m * n * 4);
    be.tensorUpload(xd, x.data(), m * k * 4);
    if (bits == 8) {
        be.opI8Prep(xd, m, k, false);
        be.opI8Gemm(yd, w.data(), ws.data(), n, false);
    } else {
        be.opI4Prep(xd, m, k);
        be.opI4Gemm(yd, packed.data(), ws.data(), n);
    }
    std::vector<float> y(m * n);
    be.tensorDownload(yd, y.data(), m * n * 4);
    double worst = 0;
    for (size_t i = 0; i < m * n; i++) {
        const double err = std::fabs((double)y[i] - sim[i]);
        const double tol = 1e-4 + 1e-3 * std::fabs(sim[i]);   // the reference's gate
        if (err > tol) worst = std::fmax(worst, err);
    }
    EXPECT(worst == 0, "int%d linear %zux%zux%zu: worst excess error %g", bits, m, n, k, worst);
    be.tensorDestroy(xd);
    be.tensorDestroy(yd);
    be.dropWeights();  // the cache is keyed by host address, and the weights are about to be freed
}

static void gguf_gemv(tpb::Backend &be, tpb::DType dt, int fmt, size_t rows, size_t cols, size_t n, unsigned seed) {
    std::mt19937 rng(seed);
    std::uniform_real_distribution<float> ux(-1.f, 1.f);
    std::vector<float> x(n * cols);
    for (auto &v : x) v = ux(rng);
    const size_t rb = tpo_gguf_row_bytes(fmt, cols);
    std::vector<uint8_t> w(rows * rb);
    for (auto &v : w) v = (uint8_t)(rng() & 0xff);
    // pin the f16 scale fields to small finite values (src/gpu/cuda/backend.zig:3356-3377)
    const size_t bb = fmt <= 1 ? (fmt == 0 ? 34 : 18) : (fmt == 2 ? 144 : fmt == 3 ? 176 : 210);
    for (size_t off = 0; off < w.size(); off += bb) {
        const size_t dpos = fmt == 4 ? off + 208 : off;
        w[dpos] = 0x66; w[dpos + 1] = 0x2A;                       // 0.05
        if (fmt == 2 || fmt == 3) { w[off + 2] = 0x1F; w[off + 3] = 0x25; }  // dmin 0.02
    }
    std::vector<float> want(n * rows);
    tpo_gguf_gemv_q8(fmt, w.data(), rows, cols, x.data(), n, 1.0f, want.data());

    tpb::DeviceBuffer xd = be.tensorCreate(n * cols * 4), yd = be.tensorCreate(n * rows * 4);
    be.tensorUpload(xd, x.data(), n * cols * 4);
    be.opGemvQuantizeX(xd, n * cols);
    be.opGemvQuantQ8N(dt, yd, w.data(), 1.0f, rows, cols, n, 0, n);
    std::vector<float> y(n * rows);
    be.tensorDownload(yd, y.data(), n * rows * 4);
    double worst = 0;
    for (size_t i = 0; i < y.size(); i++) worst = std::fmax(worst, std::fabs((double)y[i] - (double)want[i]));
    EXPECT(worst <= 2e-2, "gguf fmt %d gemv: max abs err %g (the reference's gate is 2e-2)", fmt, worst);
    be.tensorDestroy(xd);
    be.tensorDestroy(yd);
    be.dropWeights();  // the cache is keyed by host address, and `w` is about to be freed
}

// An int8 linear whose host weight outlives the call (the cache is keyed by host address), cache kept.
static void convrot_linear_keep(tpb::Backend &be, size_t m, size_t n, size_t k, unsigned seed) {
    static std::vector<std::vector<int8_t>> keep_w;
    static std::vector<std::vector<float>> keep_ws;
    std::mt19937 rng(seed);
    std::normal_distribution<float> nd(0.f, 1.f);
    std::uniform_real_distribution<float> us(1e-3f, 1e-2f);
    std::uniform_int_distribution<int> wi(-127, 127);
    std::vector<float> x(m * k);
    for (auto &v : x) v = nd(rng);
    keep_w.emplace_back(n * k);
    keep_ws.emplace_back(n);
    std::vector<int8_t> &w = keep_w.back();
    std::vector<float> &ws = keep_ws.back();
    for (auto &v : w) v = (int8_t)wi(rng);
    for (auto &v : ws) v = us(rng);
    std::vector<int8_t> q(m * k);
    std::vector<float> as(m);
    tpo_convrot_prep(x.data(), m, k, 8, q.data(), as.data(), nullptr);
    std::vector<int32_t> acc(m * n);
    tpo_igemm_s32(q.data(), w.data(), m, n, k, acc.data());
    std::vector<double> sim(m * n);
    tpo_dequant_sim(acc.data(), as.data(), ws.data(), m, n, sim.data());
    tpb::DeviceBuffer xd = be.tensorCreate(m * k * 4), yd = be.tensorCreate(m * n * 4);
    be.tensorUpload(xd, x.data(), m * k * 4);
    be.opI8Prep(xd, m, k, false);
    be.opI8Gemm(yd, w.data(), ws.data(), n, false);
    std::vector<float> y(m * n);
    be.tensorDownload(yd, y.data(), y.size() * 4);
    double worst = 0;
    for (size_t i = 0; i < y.size(); i++) worst = std::fmax(worst, std::fabs((double)y[i] - sim[i]) - 1e-3 * std::fabs(sim[i]));
    EXPECT(worst <= 1e-4, "linear under a weight budget: error beyond 1e-3 rel + 1e-4 abs by %g", worst);
    be.tensorDestroy(xd);
    be.tensorDestroy(yd);
}

// qkNorm + rope + attn against the checker; gate = 2 % of the result's norm (bf16 operands on the
// tensor cores against the f32 definition)
static void attention(tpb::Backend &be, size_t seq, size_t heads, size_t kv_heads, unsigned seed) {
    const size_t hd = 128;
    std::mt19937 rng(seed);
    std::normal_distribution<float> nd(0.f, 1.f);
    std::vector<float> q(seq * heads * hd), k(seq * kv_heads * hd), v(seq * kv_heads * hd), qn(hd), kn(hd);
    for (auto &x : q) x = nd(rng);
    for (auto &x : k) x = nd(rng);
    for (auto &x : v) x = nd(rng);
    for (auto &x : qn) x = 1.f + 0.1f * nd(rng);
    for (auto &x : kn) x = 1.f + 0.1f * nd(rng);
    std::vector<float> pos(seq * 3), freqs(2 * seq * (hd / 2));
    for (size_t p = 0; p < seq; p++) {
        pos[3 * p] = 0.f;
        pos[3 * p + 1] = (float)(p / 8);
        pos[3 * p + 2] = (float)(p % 8);
    }
    const int axes[3] = {32, 48, 48};
    const size_t sin_off = seq * (hd / 2);
    tpo_flux_freqs(pos.data(), seq, axes, 3, 10000.0, freqs.data(), freqs.data() + sin_off);
    // the checker's result
    std::vector<float> qr(q.size()), kr(k.size()), want(q.size());
    tpo_qk_norm(q.data(), seq * heads, hd, qn.data(), 1e-5f, qr.data());
    tpo_qk_norm(k.data(), seq * kv_heads, hd, kn.data(), 1e-5f, kr.data());
    tpo_rope_interleaved(qr.data(), freqs.data(), freqs.data() + sin_off, seq, heads, hd);
    tpo_rope_interleaved(kr.data(), freqs.data(), freqs.data() + sin_off, seq, kv_heads, hd);
    const float scale = 1.0f / std::sqrt((float)hd);
    tpo_attention(qr.data(), kr.data(), v.data(), seq, seq, heads, kv_heads, hd, scale, want.data());
    auto up = [&](const std::vector<float> &a) {
        tpb::DeviceBuffer d = be.tensorCreate(a.size() * 4);
        be.tensorUpload(d, a.data(), a.size() * 4);
        return d;
    };
    tpb::DeviceBuffer qd = up(q), kd = up(k), vd = up(v), qnd = up(qn), knd = up(kn), fd = up(freqs);
    tpb::DeviceBuffer od = be.tensorCreate(q.size() * 4);
    be.attention(qd, kd, vd, od, qnd, knd, fd, sin_off, seq, heads, kv_heads, hd, 1e-5f, scale);
    std::vector<float> got(q.size());
    be.tensorDownload(od, got.data(), got.size() * 4);
    double num = 0, den = 0;
    for (size_t i = 0; i < got.size(); i++) {
        num += ((double)got[i] - want[i]) * ((double)got[i] - want[i]);
        den += (double)want[i] * want[i];
    }
    const double rel = std::sqrt(num / den);
    EXPECT(rel < 2e-2, "attention seq %zu heads %zu/%zu: relative error %g", seq, heads, kv_heads, rel);
    for (tpb::DeviceBuffer d : {qd, kd, vd, qnd, knd, fd, od}) be.tensorDestroy(d);
}

// One block of the DiT step, the reference's op sequence (src/models/dit_cuda.zig:471-516) through the
// mirror, against the same sequence composed from the checker's functions.  F = 512 (4 heads x 128),
// MLP 1024, 200 tokens.  Gate: relative Frobenius error of the latents after the block (attention runs
// with bf16 operands on the tensor cores against the checker's f32: 3e-2).
struct HostLinear {
    std::vector<int8_t> w;
    std::vector<float> ws;
    size_t n, k;
};
static HostLinear make_linear(size_t n, size_t k, std::mt19937 &rng) {
    HostLinear l{std::vector<int8_t>(n * k), std::vector<float>(n), n, k};
    std::uniform_int_distribution<int> wi(-127, 127);
    std::uniform_real_distribution<float> us(1e-3f, 1e-2f);
    for (auto &v : l.w) v = (int8_t)wi(rng);
    for (auto &v : l.ws) v = us(rng);
    return l;
}
static std::vector<float> oracle_linear(const std::vector<float> &x, size_t m, const HostLinear &l) {
    std::vector<int8_t> q(m * l.k);
    std::vector<float> as(m);
    tpo_convrot_prep(x.data(), m, l.k, 8, q.data(), as.data(), nullptr);
    std::vector<int32_t> acc(m * l.n);
    tpo_igemm_s32(q.data(), l.w.data(), m, l.n, l.k, acc.data());
    std::vector<double> sim(m * l.n);
    tpo_dequant_sim(acc.data(), as.data(), l.ws.data(), m, l.n, sim.data());
    return std::vector<float>(sim.begin(), sim.end());
}
static void dit_block(tpb::Backend &be, unsigned seed) {
    const size_t F = 512, MLPD = 1024, seq = 200, heads = 4, hd = 128;
    const float eps = 1e-5f, attn_scale = 1.0f / std::sqrt((float)hd);
    std::mt19937 rng(seed);
    std::normal_distribution<float> nd(0.f, 1.f);
    HostLinear wq = make_linear(F, F, rng), wk = make_linear(F, F, rng), wv = make_linear(F, F, rng),
               gate = make_linear(F, F, rng), wo = make_linear(F, F, rng), mlp_gate = make_linear(MLPD, F, rng),
               mlp_up = make_linear(MLPD, F, rng), mlp_down = make_linear(F, MLPD, rng);
    std::vector<float> x(seq * F), mod(6 * F), qn(hd), kn(hd);
    for (auto &v : x) v = nd(rng);
    for (size_t i = 0; i < mod.size(); i++) mod[i] = 0.1f * nd(rng) + ((i / F) % 3 == 0 ? 1.0f : 0.0f);  // premul rows ~ 1
    for (auto &v : qn) v = 1.f + 0.1f * nd(rng);
    for (auto &v : kn) v = 1.f + 0.1f * nd(rng);
    std::vector<float> pos(seq * 3), freqs(2 * seq * (hd / 2));
    for (size_t p = 0; p < seq; p++) {
        pos[3 * p] = 0.f;
        pos[3 * p + 1] = (float)(p / 16);
        pos[3 * p + 2] = (float)(p % 16);
    }
    const int axes[3] = {32, 48, 48};
    const size_t sin_off = seq * (hd / 2);
    tpo_flux_freqs(pos.data(), seq, axes, 3, 10000.0, freqs.data(), freqs.data() + sin_off);

    // ---- the checker's block ----
    std::vector<float> want = x, t1(seq * F);
    tpo_rms_mod(want.data(), seq, F, mod.data(), mod.data() + F, eps, t1.data());
    std::vector<float> q = oracle_linear(t1, seq, wq), k = oracle_linear(t1, seq, wk), v = oracle_linear(t1, seq, wv),
                       g = oracle_linear(t1, seq, gate);
    std::vector<float> qr(q.size()), kr(k.size()), att(q.size());
    tpo_qk_norm(q.data(), seq * heads, hd, qn.data(), eps, qr.data());
    tpo_qk_norm(k.data(), seq * heads, hd, kn.data(), eps, kr.data());
    tpo_rope_interleaved(qr.data(), freqs.data(), freqs.data() + sin_off, seq, heads, hd);
    tpo_rope_interleaved(kr.data(), freqs.data(), freqs.data() + sin_off, seq, heads, hd);
    tpo_attention(qr.data(), kr.data(), v.data(), seq, seq, heads, heads, hd, attn_scale, att.data());
    std::vector<float> ag(att.size());
    tpo_sigmoid_mul(att.data(), g.data(), att.size(), ag.data());
    std::vector<float> o = oracle_linear(ag, seq, wo), x1(seq * F);
    tpo_gated_add(want.data(), o.data(), mod.data() + 2 * F, seq, F, x1.data());
    tpo_rms_mod(x1.data(), seq, F, mod.data() + 3 * F, mod.data() + 4 * F, eps, t1.data());
    std::vector<float> mg = oracle_linear(t1, seq, mlp_gate), mu = oracle_linear(t1, seq, mlp_up), act(mg.size());
    tpo_silu_mul(mg.data(), mu.data(), mg.size(), act.data());
    std::vector<float> dn = oracle_linear(act, seq, mlp_down);
    tpo_gated_add(x1.data(), dn.data(), mod.data() + 5 * F, seq, F, want.data());

    // ---- the same calls through the mirror (dit_cuda.zig:471-516) ----
    auto up = [&](const std::vector<float> &a) {
        tpb::DeviceBuffer d = be.tensorCreate(a.size() * 4);
        be.tensorUpload(d, a.data(), a.size() * 4);
        return d;
    };
    tpb::DeviceBuffer x_d = up(x), mv_d = up(mod), qn_d = up(qn), kn_d = up(kn), freqs_d = up(freqs);
    tpb::DeviceBuffer t1_d = be.tensorCreate(seq * F * 4), q_d = be.tensorCreate(seq * F * 4), k_d = be.tensorCreate(seq * F * 4),
                      v_d = be.tensorCreate(seq * F * 4), g_d = be.tensorCreate(seq * F * 4), attn_d = be.tensorCreate(seq * F * 4),
                      mg_d = be.tensorCreate(seq * MLPD * 4), mu_d = be.tensorCreate(seq * MLPD * 4);
    auto lin = [&](tpb::DeviceBuffer y, const HostLinear &l) { be.opI8Gemm(y, l.w.data(), l.ws.data(), l.n, false); };
    be.rmsMod(x_d, t1_d, mv_d, seq, F, 0, F, eps);
    be.opI8Prep(t1_d, seq, F, false);                        // linPrep: one prep, four GEMMs
    lin(q_d, wq);
    lin(k_d, wk);
    lin(v_d, wv);
    lin(g_d, gate);
    be.attention(q_d, k_d, v_d, attn_d, qn_d, kn_d, freqs_d, sin_off, seq, heads, heads, hd, eps, attn_scale);
    be.sigmoidMul(attn_d, g_d, seq * F);
    be.opI8Prep(attn_d, seq, F, false);
    lin(t1_d, wo);
    be.gatedAdd(x_d, t1_d, mv_d, seq * F, F, 2 * F);
    be.rmsMod(x_d, t1_d, mv_d, seq, F, 3 * F, 4 * F, eps);
    be.opI8Prep(t1_d, seq, F, false);
    lin(mg_d, mlp_gate);
    lin(mu_d, mlp_up);
    be.siluMul(mg_d, mu_d, seq * MLPD);
    be.opI8Prep(mg_d, seq, MLPD, false);
    lin(t1_d, mlp_down);
    be.gatedAdd(x_d, t1_d, mv_d, seq * F, F, 5 * F);
    std::vector<float> got(seq * F);
    be.tensorDownload(x_d, got.data(), got.size() * 4);

    // ---- the block again with the producers folded into the preps and the gated residuals into the
    // GEMM epilogues: same arithmetic, one FMA contraction in the residual ----
    // No host synchronisation anywhere in this sequence: every kernel is launched while its predecessor
    // still runs (programmatic dependent launch), so a kernel that read its input ahead of
    // griddepcontrol.wait would show up here as a wrong residual.
    be.tensorUpload(x_d, x.data(), x.size() * 4);
    be.prepRmsMod(x_d, mv_d, seq, F, 0, F, eps);
    lin(q_d, wq);
    lin(k_d, wk);
    lin(v_d, wv);
    lin(g_d, gate);
    be.attention(q_d, k_d, v_d, attn_d, qn_d, kn_d, freqs_d, sin_off, seq, heads, heads, hd, eps, attn_scale);
    be.prepSigmoidMul(attn_d, g_d, seq, F);
    be.gemmGatedAdd(x_d, wo.w.data(), wo.ws.data(), F, mv_d, 2 * F);
    be.prepRmsMod(x_d, mv_d, seq, F, 3 * F, 4 * F, eps);
    lin(mg_d, mlp_gate);
    lin(mu_d, mlp_up);
    be.prepSiluMul(mg_d, mu_d, seq, MLPD);
    be.gemmGatedAdd(x_d, mlp_down.w.data(), mlp_down.ws.data(), F, mv_d, 5 * F);
    std::vector<float> fused(seq * F);
    be.tensorDownload(x_d, fused.data(), fused.size() * 4);
    double fnum = 0, fden = 0;
    for (size_t i = 0; i < got.size(); i++) {
        fnum += ((double)fused[i] - got[i]) * ((double)fused[i] - got[i]);
        fden += (double)got[i] * got[i];
    }
    EXPECT(std::sqrt(fnum / fden) < 1e-4, "dit block, fused against the reference sequence: relative error %g", std::sqrt(fnum / fden));

    // ---- and with the MLP's gate and up projections in one launch, the SiLU gate in its epilogue, then a
    // plain prep, and q, k, v and gate in one launch too: the bits of the fused block above (f32: the same
    // arithmetic in the same order) ----
    be.tensorUpload(x_d, x.data(), x.size() * 4);
    be.prepRmsMod(x_d, mv_d, seq, F, 0, F, eps);
    {
        const tpb::DeviceBuffer ys[4] = {q_d, k_d, v_d, g_d};
        const void *ws[4] = {wq.w.data(), wk.w.data(), wv.w.data(), gate.w.data()};
        const float *sc[4] = {wq.ws.data(), wk.ws.data(), wv.ws.data(), gate.ws.data()};
        be.gemmGroup(4, ys, ws, sc, F);
    }
    be.attention(q_d, k_d, v_d, attn_d, qn_d, kn_d, freqs_d, sin_off, seq, heads, heads, hd, eps, attn_scale);
    be.prepSigmoidMul(attn_d, g_d, seq, F);
    be.gemmGatedAdd(x_d, wo.w.data(), wo.ws.data(), F, mv_d, 2 * F);
    be.prepRmsMod(x_d, mv_d, seq, F, 3 * F, 4 * F, eps);
    be.gemmSiluPair(mg_d, mlp_gate.w.data(), mlp_gate.ws.data(), mlp_up.w.data(), mlp_up.ws.data(), MLPD);
    be.opI8Prep(mg_d, seq, MLPD, false);
    be.gemmGatedAdd(x_d, mlp_down.w.data(), mlp_down.ws.data(), F, mv_d, 5 * F);
    std::vector<float> paired(seq * F);
    be.tensorDownload(x_d, paired.data(), paired.size() * 4);
    size_t pair_diff = 0;
    for (size_t i = 0; i < paired.size(); i++) pair_diff += std::memcmp(&paired[i], &fused[i], 4) != 0;
    EXPECT(pair_diff == 0, "dit block, paired MLP and grouped projections against the fused block: %zu of %zu values differ", pair_diff, paired.size());

    double num = 0, den = 0, moved = 0;
    for (size_t i = 0; i < got.size(); i++) {
        num += ((double)got[i] - want[i]) * ((double)got[i] - want[i]);
        den += (double)want[i] * want[i];
        moved += ((double)want[i] - x[i]) * ((double)want[i] - x[i]);
    }
    EXPECT(std::sqrt(num / den) < 3e-2, "dit block: relative error %g", std::sqrt(num / den));
    EXPECT(moved > 0, "dit block: the block did not change the latents");
    for (tpb::DeviceBuffer d : {x_d, mv_d, qn_d, kn_d, freqs_d, t1_d, q_d, k_d, v_d, g_d, attn_d, mg_d, mu_d}) be.tensorDestroy(d);
    be.dropWeights();
}

// Forty prep + GEMM pairs issued as fast as the host can, alternating between two activations, no
// synchronisation until the end: each output must be bit-identical to the one obtained with a
// synchronisation after every call (a GEMM that picked up the scales or the quantised rows of the
// previous iteration, or read them before its dependency wait, differs).
static void launch_order(tpb::Backend &be, unsigned seed) {
    const size_t m = 300, k = 1024, n = 512, iters = 40;
    std::mt19937 rng(seed);
    std::normal_distribution<float> nd(0.f, 1.f);
    static HostLinear lin = make_linear(n, k, rng);          // outlives the call: the cache is keyed by address
    std::vector<float> x0(m * k), x1(m * k);
    for (auto &v : x0) v = nd(rng);
    for (auto &v : x1) v = 7.f * nd(rng);
    tpb::DeviceBuffer xd[2] = {be.tensorCreate(m * k * 4), be.tensorCreate(m * k * 4)};
    be.tensorUpload(xd[0], x0.data(), m * k * 4);
    be.tensorUpload(xd[1], x1.data(), m * k * 4);
    std::vector<float> ref[2] = {std::vector<float>(m * n), std::vector<float>(m * n)};
    tpb::DeviceBuffer yd = be.tensorCreate(iters * m * n * 4);
    for (int s = 0; s < 2; s++) {
        be.opI8Prep(xd[s], m, k, false);
        be.opI8Gemm(yd, lin.w.data(), lin.ws.data(), n, false);
        be.tensorDownload(yd, ref[s].data(), m * n * 4);     // synchronises
    }
    for (size_t i = 0; i < iters; i++) {
        tpb::DeviceBuffer yi;
        yi.p = static_cast<char *>(yd.p) + i * m * n * 4;
        yi.size = m * n * 4;
        be.opI8Prep(xd[i & 1], m, k, false);
        be.opI8Gemm(yi, lin.w.data(), lin.ws.data(), n, false);
    }
    std::vector<float> all(iters * m * n);
    be.tensorDownload(yd, all.data(), all.size() * 4);
    size_t bad = 0;
    for (size_t i = 0; i < iters; i++)
        if (std::memcmp(all.data() + i * m * n, ref[i & 1].data(), m * n * 4) != 0) bad++;
    EXPECT(bad == 0, "launch order: %zu of %zu back-to-back linears differ from the synchronised result", bad, iters);
    be.tensorDestroy(xd[0]);
    be.tensorDestroy(xd[1]);
    be.tensorDestroy(yd);
    be.dropWeights();
}

int main() {
    try {
        tpb::Backend be(0);
        convrot_linear(be, 8, 256, 384, 512, 1);
        convrot_linear(be, 4, 130, 272, 768, 2);
        convrot_linear(be, 8, 300, 3072, 256, 3);
        // the reference's grouped GEMV test shape: rows 24, cols 512, 5 activation rows
        gguf_gemv(be, tpb::DType::q8_0, 0, 24, 512, 5, 271);
        gguf_gemv(be, tpb::DType::q4_0, 1, 24, 512, 5, 272);
        gguf_gemv(be, tpb::DType::q4_k, 2, 24, 512, 5, 314);
        gguf_gemv(be, tpb::DType::q5_k, 3, 24, 512, 5, 315);
        gguf_gemv(be, tpb::DType::q6_k, 4, 24, 512, 5, 316);

        attention(be, 200, 4, 2, 401);
        attention(be, 384, 2, 2, 402);
        dit_block(be, 501);
        launch_order(be, 601);

        // weights under a budget (--vram-budget): 300 x 3072 int8 = 0.92 MB per weight under 2 MB: the
        // third linear evicts the first weight and the results stay right
        be.setWeightBudget(2u << 20);
        convrot_linear_keep(be, 300, 3072, 256, 31);
        convrot_linear_keep(be, 300, 3072, 256, 32);
        convrot_linear_keep(be, 300, 3072, 256, 33);
        EXPECT(be.weightEvictions() > 0 && be.weightBytes() <= (2u << 20), "budget: %zu evictions, %zu bytes cached",
               be.weightEvictions(), be.weightBytes());
        bool full = false;
        try {
            std::vector<int8_t> huge(3u << 20);
            be.cachedWeight(huge.data(), huge.size());
        } catch (const tpb::Error &e) {
            full = e.status == TPB_ERR_OOM;
        }
        EXPECT(full, "a weight larger than the budget must fail with TPB_ERR_OOM");
        be.dropWeights();
        be.setWeightBudget(0);

        // error behaviour: a GEMM without its prep, a width the rotation cannot take
        tpb::DeviceBuffer t = be.tensorCreate(1 << 16);
        std::vector<int8_t> w(256 * 256);
        std::vector<float> ws(256, 1.f);
        bool threw = false;
        try {
            be.opI4Gemm(t, w.data(), ws.data(), 256);   // last prep was int8
        } catch (const tpb::Error &e) {
            threw = e.status == TPB_ERR_STATE;
        }
        EXPECT(threw, "opI4Gemm after an int8 prep must fail with TPB_ERR_STATE");
        threw = false;
        try {
            be.opI8Prep(t, 4, 250, false);
        } catch (const tpb::Error &e) {
            threw = e.status == TPB_ERR_INVALID_ARG;
        }
        EXPECT(threw, "opI8Prep with cols %% 256 != 0 must fail with TPB_ERR_INVALID_ARG");
        be.sync();
        be.tensorDestroy(t);
    } catch (const tpb::Error &e) {
        std::printf("FAIL: exception %d: %s\n", e.status, e.what());
        return 1;
    }
    if (failures == 0) std::printf("OK\n");
    return failures ? 1 : 0;
}
