// TEST INFRASTRUCTURE. Exercises the operator-level C++ mirror (blackforge_b200/csrc/host/bfb200.hpp, namespace
// bfb200) directly from C++: the bf16 / e4m3 operator forms and the DeviceTensor mechanics that Model does not go
// through. Expected values are evaluated here in double precision from the same inputs (the definitions of
// src/backend/cpu/ops.cpp: matmul, linear, rmsnorm with eps 1e-6, silu feed-forward with residual, causal
// multi-head attention with scale 1/sqrt(head_dim)), with the operands rounded to bf16 where the operator rounds
// them. Exit code 0 = every check passed.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../blackforge_b200/csrc/host/bfb200.hpp"

using namespace bfb200;

namespace {

int failures = 0;

void expect(bool ok, const std::string& what) {
    if (!ok) {
        ++failures;
        std::printf("FAILED: %s\n", what.c_str());
    }
}

float bf16Round(float x) {
    uint32_t u;
    std::memcpy(&u, &x, 4);
    u = (u + 0x7FFFu + ((u >> 16) & 1u)) & 0xFFFF0000u;
    std::memcpy(&x, &u, 4);
    return x;
}

HostTensor ramp(std::vector<std::size_t> shape, float scale, float shift, bool rounded = true) {
    HostTensor t;
    t.shape = std::move(shape);
    t.data.resize(t.elementCount());
    for (std::size_t i = 0; i < t.data.size(); ++i) {
        const float v = scale * static_cast<float>((i * 37 + 11) % 29) / 29.0f + shift;
        t.data[i] = rounded ? bf16Round(v) : v;
    }
    return t;
}

void near(const std::vector<double>& want, const HostTensor& got, double tol, const std::string& what) {
    if (want.size() != got.data.size()) {
        expect(false, what + ": sizes differ");
        return;
    }
    double worst = 0.0, scale = 1e-30;
    for (std::size_t i = 0; i < want.size(); ++i) {
        worst = std::fmax(worst, std::fabs(want[i] - got.data[i]));
        scale = std::fmax(scale, std::fabs(want[i]));
    }
    std::printf("%-46s max abs diff / max abs %.3g (bar %.1g)\n", what.c_str(), worst / scale, tol);
    expect(worst / scale <= tol, what);
}

std::vector<double> matmulRef(const HostTensor& a, const HostTensor& b, std::size_t m, std::size_t k, std::size_t n) {
    std::vector<double> c(m * n, 0.0);
    for (std::size_t i = 0; i < m; ++i)
        for (std::size_t j = 0; j < n; ++j) {
            double acc = 0.0;
            for (std::size_t p = 0; p < k; ++p) acc += static_cast<double>(a.data[i * k + p]) * b.data[p * n + j];
            c[i * n + j] = acc;
        }
    return c;
}

std::vector<double> rmsnormRef(const std::vector<double>& x, std::size_t rows, std::size_t d) {
    std::vector<double> out(x.size());
    for (std::size_t r = 0; r < rows; ++r) {
        double ss = 0.0;
        for (std::size_t i = 0; i < d; ++i) ss += x[r * d + i] * x[r * d + i];
        const double inv = 1.0 / std::sqrt(ss / static_cast<double>(d) + 1e-6);
        for (std::size_t i = 0; i < d; ++i) out[r * d + i] = x[r * d + i] * inv;
    }
    return out;
}

std::vector<double> toDouble(const HostTensor& t) { return std::vector<double>(t.data.begin(), t.data.end()); }

std::vector<double> gemmRef(const std::vector<double>& a, const HostTensor& w, std::size_t m, std::size_t k, std::size_t n) {
    std::vector<double> c(m * n, 0.0);
    for (std::size_t i = 0; i < m; ++i)
        for (std::size_t j = 0; j < n; ++j) {
            double acc = 0.0;
            for (std::size_t p = 0; p < k; ++p) acc += a[i * k + p] * w.data[p * n + j];
            c[i * n + j] = acc;
        }
    return c;
}

// causal attention core on [batch, len, dim] with `old` cached positions before the `q` rows
std::vector<double> attentionRef(const std::vector<double>& q, const std::vector<double>& k, const std::vector<double>& v,
                                 std::size_t batch, std::size_t newLen, std::size_t totalLen, std::size_t dim, std::size_t heads) {
    const std::size_t hd = dim / heads, old = totalLen - newLen;
    const double scale = 1.0 / std::sqrt(static_cast<double>(hd));
    std::vector<double> out(batch * newLen * dim, 0.0);
    for (std::size_t b = 0; b < batch; ++b)
        for (std::size_t h = 0; h < heads; ++h)
            for (std::size_t i = 0; i < newLen; ++i) {
                const std::size_t visible = old + i + 1;
                std::vector<double> sc(visible);
                double m = -1e300, l = 0.0;
                for (std::size_t j = 0; j < visible; ++j) {
                    double dot = 0.0;
                    for (std::size_t d = 0; d < hd; ++d) dot += q[(b * newLen + i) * dim + h * hd + d] * k[(b * totalLen + j) * dim + h * hd + d];
                    sc[j] = dot * scale;
                    m = std::fmax(m, sc[j]);
                }
                for (std::size_t j = 0; j < visible; ++j) {
                    sc[j] = std::exp(sc[j] - m);
                    l += sc[j];
                }
                for (std::size_t j = 0; j < visible; ++j)
                    for (std::size_t d = 0; d < hd; ++d)
                        out[(b * newLen + i) * dim + h * hd + d] += sc[j] / l * v[(b * totalLen + j) * dim + h * hd + d];
            }
    return out;
}

// gradients of sum(g * attention(q, k, v)) in double, straight from the definition: p = softmax row, dS = p (dP - D)
struct GradRef {
    std::vector<double> dq, dk, dv;
};
GradRef attentionBackwardRef(const std::vector<double>& g, const std::vector<double>& q, const std::vector<double>& k,
                             const std::vector<double>& v, std::size_t batch, std::size_t newLen, std::size_t totalLen,
                             std::size_t dim, std::size_t heads) {
    const std::size_t hd = dim / heads, old = totalLen - newLen;
    const double scale = 1.0 / std::sqrt(static_cast<double>(hd));
    GradRef r{std::vector<double>(q.size(), 0.0), std::vector<double>(k.size(), 0.0), std::vector<double>(v.size(), 0.0)};
    for (std::size_t b = 0; b < batch; ++b)
        for (std::size_t h = 0; h < heads; ++h)
            for (std::size_t i = 0; i < newLen; ++i) {
                const std::size_t visible = old + i + 1, qi = (b * newLen + i) * dim + h * hd;
                std::vector<double> p(visible), dp(visible);
                double m = -1e300, l = 0.0, dTerm = 0.0;
                for (std::size_t j = 0; j < visible; ++j) {
                    const std::size_t kj = (b * totalLen + j) * dim + h * hd;
                    double dot = 0.0, dpv = 0.0;
                    for (std::size_t d = 0; d < hd; ++d) {
                        dot += q[qi + d] * k[kj + d];
                        dpv += g[qi + d] * v[kj + d];
                    }
                    p[j] = dot * scale;
                    dp[j] = dpv;
                    m = std::fmax(m, p[j]);
                }
                for (std::size_t j = 0; j < visible; ++j) {
                    p[j] = std::exp(p[j] - m);
                    l += p[j];
                }
                for (std::size_t j = 0; j < visible; ++j) {
                    p[j] /= l;
                    dTerm += p[j] * dp[j];
                }
                for (std::size_t j = 0; j < visible; ++j) {
                    const std::size_t kj = (b * totalLen + j) * dim + h * hd;
                    const double ds = p[j] * (dp[j] - dTerm) * scale;
                    for (std::size_t d = 0; d < hd; ++d) {
                        r.dq[qi + d] += ds * k[kj + d];
                        r.dk[kj + d] += ds * q[qi + d];
                        r.dv[kj + d] += p[j] * g[qi + d];
                    }
                }
            }
    return r;
}

}  // namespace

int main() {
    // ---- DeviceTensor mechanics (device_tensor.cu:19-117) ----
    {
        HostTensor a = ramp({6, 10}, 1.0f, -0.5f);
        DeviceTensor da = DeviceTensor::fromHost(a);
        DeviceTensor c = da.clone();
        expect(c.data() != da.data() && c.toHost().data == a.data, "clone copies into its own buffer");
        float* before = c.data();
        DeviceTensor r = std::move(c).reshaped({10, 6});
        expect(r.data() == before && r.shape() == std::vector<std::size_t>({10, 6}) && c.data() == nullptr, "reshaped() && keeps the buffer, empties the source");
        DeviceTensor moved(std::move(r));
        expect(r.data() == nullptr && moved.data() == before, "move construction");
        DeviceTensor target = DeviceTensor::zeros({3, 3});
        target = std::move(moved);
        expect(target.data() == before && moved.data() == nullptr && target.elementCount() == 60, "move assignment");
        bool threw = false;
        try {
            (void)std::move(target).reshaped({7, 7});
        } catch (const std::invalid_argument&) {
            threw = true;
        }
        expect(threw, "reshaped() to another element count throws std::invalid_argument");
        const HostTensor z = DeviceTensor::zeros({4, 5}).toHost();
        bool allZero = true;
        for (float v : z.data) allZero = allZero && v == 0.0f;
        expect(allZero && z.shape == std::vector<std::size_t>({4, 5}), "zeros");
    }
    // ---- GEMM forms (ops_tensorcore.cu:308-348) ----
    const std::size_t m = 96, k = 160, n = 72;
    HostTensor a = ramp({m, k}, 1.0f, -0.5f), w = ramp({k, n}, 0.6f, -0.3f), bias = ramp({n}, 0.4f, -0.2f, false);
    DeviceTensor da = DeviceTensor::fromHost(a), dw = DeviceTensor::fromHost(w), dbias = DeviceTensor::fromHost(bias);
    const std::vector<double> prod = matmulRef(a, w, m, k, n);
    near(prod, matmulBf16(da, dw).toHost(), 1e-5, "matmulBf16 (bf16-exact operands)");
    near(prod, matmulBf16CachedWeight(da, dw).toHost(), 1e-5, "matmulBf16CachedWeight");
    {
        // the cache is keyed by the weight tensor: new values in the same buffer need an invalidation
        HostTensor w2 = ramp({k, n}, -0.5f, 0.25f);
        DeviceTensor dw2 = DeviceTensor::fromHost(w2);
        near(matmulRef(a, w2, m, k, n), matmulBf16CachedWeight(da, dw2).toHost(), 1e-5, "matmulBf16CachedWeight, second weight");
        invalidateBf16WeightCache();
        near(prod, matmulBf16CachedWeight(da, dw).toHost(), 1e-5, "matmulBf16CachedWeight after invalidation");
    }
    near(prod, matmulFp8(da, dw).toHost(), 8e-2, "matmulFp8 (e4m3 operands, per-tensor scales)");
    {
        std::vector<double> lin = prod;
        for (std::size_t i = 0; i < m; ++i)
            for (std::size_t j = 0; j < n; ++j) lin[i * n + j] += bias.data[j];
        DeviceTensor x3 = DeviceTensor::fromHost(a);
        near(lin, linearBf16(std::move(x3).reshaped({4, 24, k}), dw, dbias).toHost(), 1e-5, "linearBf16 on [4, 24, 160]");
    }
    bool threw = false;
    try {
        (void)matmulBf16(da, da);
    } catch (const std::invalid_argument&) {
        threw = true;
    }
    expect(threw, "matmulBf16 with mismatched shapes throws std::invalid_argument");

    // ---- blocks: dim 256 = 2 heads of 128 (the tensor-core attention kernel), hidden 384 ----
    const std::size_t batch = 2, seq = 40, d = 256, f = 384, heads = 2;
    HostTensor x = ramp({batch, seq, d}, 1.0f, -0.5f, false), wq = ramp({d, d}, 0.12f, -0.06f), wk = ramp({d, d}, 0.10f, -0.05f),
               wv = ramp({d, d}, 0.08f, -0.04f), wo = ramp({d, d}, 0.10f, -0.05f), w1 = ramp({d, f}, 0.10f, -0.05f),
               b1 = ramp({f}, 0.2f, -0.1f, false), w2 = ramp({f, d}, 0.08f, -0.04f), b2 = ramp({d}, 0.1f, -0.05f, false);
    auto dev = [](const HostTensor& t) { return DeviceTensor::fromHost(t); };
    DeviceTensor dx = dev(x), dwq = dev(wq), dwk = dev(wk), dwv = dev(wv), dwo = dev(wo), dw1 = dev(w1), db1 = dev(b1), dw2 = dev(w2),
                 db2 = dev(b2);
    const std::size_t rows = batch * seq;
    const std::vector<double> xd = toDouble(x), normed = rmsnormRef(xd, rows, d);
    {
        std::vector<double> h = gemmRef(normed, w1, rows, d, f);
        for (std::size_t i = 0; i < rows; ++i)
            for (std::size_t j = 0; j < f; ++j) {
                const double z = h[i * f + j] + b1.data[j];
                h[i * f + j] = z / (1.0 + std::exp(-z));
            }
        std::vector<double> out = gemmRef(h, w2, rows, f, d);
        for (std::size_t i = 0; i < rows; ++i)
            for (std::size_t j = 0; j < d; ++j) out[i * d + j] += b2.data[j] + xd[i * d + j];
        near(out, feedForwardBf16(dx, dw1, db1, dw2, db2).toHost(), 2e-2, "feedForwardBf16");
    }
    const std::vector<double> q = gemmRef(normed, wq, rows, d, d), kk = gemmRef(normed, wk, rows, d, d), vv = gemmRef(normed, wv, rows, d, d);
    std::vector<double> attnOut;
    {
        const std::vector<double> ctx = attentionRef(q, kk, vv, batch, seq, seq, d, heads);
        attnOut = gemmRef(ctx, wo, rows, d, d);
        for (std::size_t i = 0; i < attnOut.size(); ++i) attnOut[i] += xd[i];
        near(attnOut, selfAttentionBf16(dx, dwq, dwk, dwv, dwo, heads).toHost(), 2e-2, "selfAttentionBf16");
    }
    {
        // the same sequence in pieces of 25, 1 and 14 positions through the operator-level cache
        KVCache cache;
        std::vector<float> got(rows * d, 0.0f);
        std::size_t pos = 0;
        for (std::size_t piece : {std::size_t(25), std::size_t(1), std::size_t(14)}) {
            HostTensor part;
            part.shape = {batch, piece, d};
            part.data.resize(batch * piece * d);
            for (std::size_t b = 0; b < batch; ++b)
                std::memcpy(&part.data[b * piece * d], &x.data[(b * seq + pos) * d], piece * d * sizeof(float));
            const HostTensor out = selfAttentionIncrementalBf16(dev(part), dwq, dwk, dwv, dwo, heads, cache).toHost();
            for (std::size_t b = 0; b < batch; ++b)
                std::memcpy(&got[(b * seq + pos) * d], &out.data[b * piece * d], piece * d * sizeof(float));
            pos += piece;
            expect(cache.length == pos, "cache length after a piece");
        }
        HostTensor gotT;
        gotT.shape = {batch, seq, d};
        gotT.data = got;
        near(attnOut, gotT, 2e-2, "selfAttentionIncrementalBf16 (25 + 1 + 14)");
    }
    {
        // the bf16 attention core alone, with 8 cached positions: output and row statistics
        const std::size_t newLen = 32, old = 8;
        HostTensor hq = ramp({batch, newLen, d}, 1.0f, -0.5f), hk = ramp({batch, newLen + old, d}, 0.9f, -0.45f),
                   hv = ramp({batch, newLen + old, d}, 0.8f, -0.4f);
        const float scale = 1.0f / std::sqrt(128.0f);
        FusedAttentionForwardResult r = fusedAttentionForwardBf16(dev(hq), dev(hk), dev(hv), heads, scale, old);
        near(attentionRef(toDouble(hq), toDouble(hk), toDouble(hv), batch, newLen, newLen + old, d, heads), r.output.toHost(), 1.2e-2,
             "fusedAttentionForwardBf16 with 8 cached positions");
        const HostTensor lo = r.l.toHost();
        bool sane = lo.shape == std::vector<std::size_t>({batch, heads, newLen});
        for (float v : lo.data) sane = sane && v >= 1.0f - 1e-3f && std::isfinite(v);
        expect(sane, "row sums are [batch, heads, new_len] and at least 1");
    }
    {
        // gradient of the attention core from the forward's own output and statistics: the fp32 route and the bf16
        // tensor-core route (fused_attention.hpp:59-76), 150 new rows after 40 cached ones
        const std::size_t newLen = 150, old = 40;
        HostTensor hq = ramp({batch, newLen, d}, 1.0f, -0.5f), hk = ramp({batch, newLen + old, d}, 0.9f, -0.45f),
                   hv = ramp({batch, newLen + old, d}, 0.8f, -0.4f), hg = ramp({batch, newLen, d}, 0.7f, -0.3f);
        const float scale = 1.0f / std::sqrt(128.0f);
        const GradRef want = attentionBackwardRef(toDouble(hg), toDouble(hq), toDouble(hk), toDouble(hv), batch, newLen,
                                                  newLen + old, d, heads);
        DeviceTensor dq = dev(hq), dk = dev(hk), dv = dev(hv), dg = dev(hg);
        FusedAttentionForwardResult f = fusedAttentionForward(dq, dk, dv, heads, scale, old);
        FusedAttentionGrad g32 = fusedAttentionBackward(dg, dq, dk, dv, f.output, f.m, f.l, heads, scale, old);
        near(want.dq, g32.dQ.toHost(), 2e-4, "fusedAttentionBackward dQ");
        near(want.dk, g32.dK.toHost(), 2e-4, "fusedAttentionBackward dK");
        near(want.dv, g32.dV.toHost(), 2e-4, "fusedAttentionBackward dV");
        FusedAttentionGrad g16 = fusedAttentionBackwardBf16(dg, dq, dk, dv, f.output, f.m, f.l, heads, scale, old);
        near(want.dq, g16.dQ.toHost(), 1e-2, "fusedAttentionBackwardBf16 dQ");
        near(want.dk, g16.dK.toHost(), 1e-2, "fusedAttentionBackwardBf16 dK");
        near(want.dv, g16.dV.toHost(), 1e-2, "fusedAttentionBackwardBf16 dV");
        bool threw = false;
        try {
            fusedAttentionBackward(dg, dq, dk, dv, f.output, f.m, f.l, heads, scale, old + 1);
        } catch (const std::invalid_argument&) {
            threw = true;
        }
        expect(threw, "fusedAttentionBackward rejects old_len + new_len != total_len");
    }
    {
        // gradients of C = A B on the bf16 route (autodiff.hpp:18-37), plain and with the cached weight copy
        const std::size_t m = 192, k = 256, n = 128;
        HostTensor ha = ramp({m, k}, 1.0f, -0.5f), hb = ramp({k, n}, 0.9f, -0.45f), hg = ramp({m, n}, 0.8f, -0.4f);
        std::vector<double> wantA(m * k, 0.0), wantB(k * n, 0.0);
        for (std::size_t i = 0; i < m; ++i)
            for (std::size_t j = 0; j < n; ++j) {
                const double gv = hg.data[i * n + j];
                for (std::size_t p = 0; p < k; ++p) {
                    wantA[i * k + p] += gv * hb.data[p * n + j];
                    wantB[p * n + j] += gv * ha.data[i * k + p];
                }
            }
        DeviceTensor da = dev(ha), db = dev(hb), dg = dev(hg);
        MatmulGrad g1 = matmulBf16Backward(da, db, dg);
        near(wantA, g1.dA.toHost(), 2e-5, "matmulBf16Backward dA");
        near(wantB, g1.dB.toHost(), 2e-5, "matmulBf16Backward dB");
        MatmulGrad g2 = matmulBf16BackwardCachedWeight(da, db, dg);
        MatmulGrad g3 = matmulBf16BackwardCachedWeight(da, db, dg);   // second call: the cached copy
        near(wantA, g2.dA.toHost(), 2e-5, "matmulBf16BackwardCachedWeight dA");
        near(wantB, g3.dB.toHost(), 2e-5, "matmulBf16BackwardCachedWeight dB (cache hit)");
        invalidateBf16WeightCache();
        bool threw = false;
        try {
            matmulBf16Backward(da, db, da);
        } catch (const std::invalid_argument&) {
            threw = true;
        }
        expect(threw, "matmulBf16Backward rejects a gradient of the wrong shape");
    }
    std::printf(failures == 0 ? "ops mirror: all checks passed\n" : "ops mirror: %d check(s) FAILED\n", failures);
    return failures == 0 ? 0 : 1;
}
