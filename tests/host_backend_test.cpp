// Exercises the C++ host mirror (puter_b200/host/backend.hpp) the way the reference's own tests exercise a device backend:
// literal fixtures from execution/math_gated_residual_intrinsic_test.go:17-65, execution/page_intrinsic_test.go:15-72 and
// device/metal/attention/multihead_parity_darwin_test.go:16-37.  Exit code 0 = all checks passed; 77 = no CUDA device.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <vector>

#include "../puter_b200/host/backend.hpp"

using namespace puter;

static int failures = 0;
#define CHECK(cond)                                                     \
    do {                                                                \
        if (!(cond)) { printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #cond); failures++; } \
    } while (0)

template <typename T> static void up(Backend& b, DeviceTensor& t, const std::vector<T>& v) { b.Upload(t, v.data(), (long long)(v.size() * sizeof(T))); }
template <typename T> static std::vector<T> down(Backend& b, DeviceTensor& t, size_t n) {
    std::vector<T> v(n);
    b.Download(v.data(), t, (long long)(n * sizeof(T)));
    return v;
}

int main() {
    Backend* backend = nullptr;
    try {
        backend = new Backend(0);
    } catch (const DeviceError& e) {
        printf("no device: [%d] %s\n", e.code, e.what());
        return e.code == -1 ? 77 : 1;
    }
    Backend& b = *backend;
    CUDADeviceRef ctx = b.Context();
    {   // gated residual known answer
        std::vector<float> res = {1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12}, br(12, 1.f);
        std::vector<float> mod = {0, 0, 0, 0, 0, 0, 0.5f, 1, 2, 0, 0, 0, 0, 0, 0, 3, 4, 5};
        DeviceTensor r(ctx, 48), bt(ctx, 48), m(ctx, 72), o(ctx, 48);
        up(b, r, res); up(b, bt, br); up(b, m, mod);
        b.GatedResidual(r.DispatchPointer(), bt.DispatchPointer(), m.DispatchPointer(), o.DispatchPointer(), 4, 3, 2, 9, 0, DType::Float32);
        auto got = down<float>(b, o, 12);
        const float want[12] = {1.5f, 3, 5, 4.5f, 6, 8, 10, 12, 14, 13, 15, 17};
        for (int i = 0; i < 12; i++) CHECK(got[i] == want[i]);
        bool threw = false;
        try { b.GatedResidual(r.DispatchPointer(), bt.DispatchPointer(), m.DispatchPointer(), o.DispatchPointer(), 4, 3, 2, 9, 1, DType::Float32); }
        catch (const DeviceError& e) { threw = e.code == -2; }
        CHECK(threw);  // modulation too narrow for set 1: the Go method panics
    }
    {   // page write / gather known answer: storage [2,3,2,1,1], layer 1
        std::vector<float> zeros(12, 0.f), vals = {7, 8};
        std::vector<int32_t> ids = {1, 1}, offs = {0, 1}, table = {1};
        DeviceTensor st(ctx, 48), v(ctx, 8), pi(ctx, 8), po(ctx, 8), pt(ctx, 4), out(ctx, 8);
        up(b, st, zeros); up(b, v, vals); up(b, pi, ids); up(b, po, offs); up(b, pt, table);
        b.KVPageWrite(st.DispatchPointer(), v.DispatchPointer(), pi.DispatchPointer(), po.DispatchPointer(), st.DispatchPointer(), 3, 2, 1, 2, 6,
                      DType::Float32);
        auto flat = down<float>(b, st, 12);
        CHECK(flat[8] == 7 && flat[9] == 8);
        b.KVPageGather(st.DispatchPointer(), pt.DispatchPointer(), out.DispatchPointer(), 3, 2, 1, 2, 6, DType::Float32);
        auto g = down<float>(b, out, 2);
        CHECK(g[0] == 7 && g[1] == 8);
        b.EndBatch();
    }
    {   // decode GQA causal known answer: q zeros [1,2*2], k zeros [3,1*2], v rows -> mean of the three live keys
        std::vector<float> q(4, 0.f), k(6, 0.f), v = {1, 10, 2, 20, 3, 30};
        DeviceTensor qt(ctx, 16), kt(ctx, 24), vt(ctx, 24), ot(ctx, 16);
        up(b, qt, q); up(b, kt, k); up(b, vt, v);
        MultiHeadAttentionConfig cfg;
        cfg.NumHeads = 2; cfg.KVHeadCount = 1; cfg.HeadDim = 2; cfg.Causal = true;
        b.MultiHeadAttention(cfg, qt.DispatchPointer(), kt.DispatchPointer(), vt.DispatchPointer(), ot.DispatchPointer(), 1, 3, DType::Float32);
        auto o = down<float>(b, ot, 4);
        const float want[4] = {2, 20, 2, 20};
        for (int i = 0; i < 4; i++) CHECK(std::fabs(o[i] - want[i]) <= 4e-6f);
    }
    {   // convert package shape: host slices, ErrLenMismatch on unequal lengths
        std::vector<float> src = {0.f, 0.5f, 1.f, 9.f, -2.5f};
        std::vector<uint16_t> dst(5);
        CHECK(convert::Float32ToBFloat16(b, dst.data(), 5, src.data(), 5));
        CHECK(dst[1] == 0x3F00 && dst[2] == 0x3F80 && dst[4] == 0xC020);
        CHECK(!convert::Float32ToBFloat16(b, dst.data(), 4, src.data(), 5));
        std::vector<float> back(5);
        CHECK(convert::BFloat16ToFloat32(b, back.data(), 5, dst.data(), 5));
        for (int i = 0; i < 5; i++) CHECK(back[i] == src[i]);
    }
    {   // shape.last_token: [2, 3, 2] -> the final row of each batch item (execution/shape_intrinsic_test.go:53-88); and the
        // device hook's byte-sized form on a [6, 4] allocation with 3 live rows (execution/bind_test.go:1201-1239)
        std::vector<float> x = {1, 2, 3, 4, 5, 6, 10, 20, 30, 40, 50, 60};
        DeviceTensor xt(ctx, 48), ot(ctx, 16);
        up(b, xt, x);
        b.LastToken(xt.DispatchPointer(), ot.DispatchPointer(), 2, 3, 2, DType::Float32);
        auto o = down<float>(b, ot, 4);
        CHECK(o[0] == 5 && o[1] == 6 && o[2] == 50 && o[3] == 60);
        std::vector<float> y = {1, 2, 3, 4, 9, 9, 9, 9, 5, 6, 7, 8, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
        DeviceTensor yt(ctx, 96);
        up(b, yt, y);
        b.IntrinsicLastToken(yt.DispatchPointer(), ot.DispatchPointer(), 3, 16, 16, DType::Float32);
        o = down<float>(b, ot, 4);
        CHECK(o[0] == 5 && o[1] == 6 && o[2] == 7 && o[3] == 8);
    }
    {   // softmax of one vector: [0, 0, 0, 0] -> quarters; log-softmax of the same -> -log(4) by the reference's FastLog32
        std::vector<float> x(4, 0.f);
        DeviceTensor xt(ctx, 16), ot(ctx, 16);
        up(b, xt, x);
        b.Softmax(ot.DispatchPointer(), xt.DispatchPointer(), 4, DType::Float32);
        auto o = down<float>(b, ot, 4);
        for (int i = 0; i < 4; i++) CHECK(o[i] == 0.25f);
        b.LogSoftmax(ot.DispatchPointer(), xt.DispatchPointer(), 4, DType::Float32);
        o = down<float>(b, ot, 4);
        for (int i = 0; i < 4; i++) CHECK(std::fabs(o[i] + 1.3862944f) <= 1e-4f);
    }
    {   // RMSNorm config validation mirrors RMSNormConfig.Validate
        DeviceTensor x(ctx, 32);
        bool threw = false;
        try { b.RMSNorm(RMSNormConfig{0.0}, x.DispatchPointer(), x.DispatchPointer(), x.DispatchPointer(), 2, 4, DType::Float32); }
        catch (const DeviceError& e) { threw = std::strstr(e.what(), "epsilon must be positive") != nullptr; }
        CHECK(threw);
    }
    delete backend;
    printf(failures ? "host backend: %d failures\n" : "host backend: all checks passed\n", failures);
    return failures ? 1 : 0;
}
