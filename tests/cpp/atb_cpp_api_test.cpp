// C++ caller of the atb:: operator API, written the way the reference's demos drive it
// (example/op_demo/paged_attention/paged_attention_demo.cpp:94-134 and
//  example/op_demo/reshape_and_cache/reshape_and_cache_demo.cpp of the reference): CreateContext,
// CreateOperation(param), Setup -> workspace size, Execute on a VariantPack, stream sync, Destroy.
//
//   atb_cpp_api_test cpu   : contract / error-code checks that need no GPU
//   atb_cpp_api_test gpu   : ReshapeAndCache + PagedAttention (GQA, fp16) against a double-precision
//                            host computation in this file
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <vector>
#include "atb/atb_infer.h"

#define CHECK(cond)                                                                   \
    do {                                                                              \
        if (!(cond)) {                                                                \
            std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);   \
            return 1;                                                                 \
        }                                                                             \
    } while (0)

static atb::Tensor MakeTensor(aclDataType dt, std::initializer_list<int64_t> dims, void *dev, void *host = nullptr)
{
    atb::Tensor t;
    t.desc.dtype = dt;
    t.desc.format = ACL_FORMAT_ND;
    t.desc.shape.dimNum = dims.size();
    int i = 0;
    for (int64_t d : dims) {
        t.desc.shape.dims[i++] = d;
    }
    t.deviceData = dev;
    t.hostData = host;
    t.dataSize = atb::Utils::GetTensorSize(t.desc);
    return t;
}

static int RunCpu()
{
    static_assert(sizeof(atb::infer::PagedAttentionParam) == 120, "ABI");
    static_assert(sizeof(atb::infer::ReshapeAndCacheParam) == 24, "ABI");
    atb::Operation *op = nullptr;
    atb::infer::PagedAttentionParam p;
    CHECK(atb::CreateOperation(p, &op) == atb::ERROR_INVALID_PARAM); // headNum == 0
    p.headNum = 8;
    p.kvHeadNum = 3;
    CHECK(atb::CreateOperation(p, &op) == atb::ERROR_INVALID_PARAM); // 8 % 3 != 0
    p.kvHeadNum = 2;
    p.rsv[3] = 1;
    CHECK(atb::CreateOperation(p, &op) == atb::ERROR_INVALID_PARAM); // reserved bytes must be zero
    p.rsv[3] = 0;
    CHECK(atb::CreateOperation(p, nullptr) == atb::ERROR_INVALID_PARAM);
    CHECK(atb::CreateOperation(p, &op) == atb::NO_ERROR && op != nullptr);
    CHECK(op->GetName() == "PagedAttentionOperation");
    CHECK(op->GetInputNum() == 5 && op->GetOutputNum() == 1);

    atb::SVector<atb::TensorDesc> inDescs, outDescs;
    void *fake = reinterpret_cast<void *>(0x1000);
    int32_t lens[2] = {5, 200};
    atb::VariantPack vp;
    vp.inTensors = {MakeTensor(ACL_FLOAT16, {2, 8, 128}, fake), MakeTensor(ACL_FLOAT16, {4, 128, 2, 128}, fake),
                    MakeTensor(ACL_FLOAT16, {4, 128, 2, 128}, fake), MakeTensor(ACL_INT32, {2, 2}, fake),
                    MakeTensor(ACL_INT32, {2}, fake, lens)};
    vp.outTensors = {MakeTensor(ACL_FLOAT16, {2, 8, 128}, fake)};
    for (size_t i = 0; i < vp.inTensors.size(); ++i) {
        inDescs.push_back(vp.inTensors.at(i).desc);
    }
    CHECK(op->InferShape(inDescs, outDescs) == atb::NO_ERROR);
    CHECK(outDescs.size() == 1 && outDescs.at(0).shape.dims[2] == 128);

    uint64_t ws = 0;
    atb::Context *ctx = nullptr;
    CHECK(atb::CreateContext(&ctx) == atb::NO_ERROR);
    CHECK(op->Execute(vp, nullptr, 0, ctx) == atb::ERROR_INVALID_PARAM); // Execute before Setup
    CHECK(op->Setup(vp, ws, nullptr) == atb::ERROR_INVALID_PARAM);       // null context
    atb::VariantPack bad = vp;
    bad.inTensors.resize(4);
    CHECK(op->Setup(bad, ws, ctx) == atb::ERROR_INVALID_IN_TENSOR_NUM);
    bad = vp;
    bad.inTensors.at(4).hostData = nullptr;
    CHECK(op->Setup(bad, ws, ctx) == atb::ERROR_INVALID_PARAM); // contextLens needs hostData
    bad = vp;
    bad.inTensors.at(1) = MakeTensor(ACL_FLOAT16, {4, 128, 256}, fake);
    CHECK(op->Setup(bad, ws, ctx) == atb::ERROR_INVALID_TENSOR_DIM_NUM);
    bad = vp;
    bad.inTensors.at(1).desc.dtype = ACL_INT8;
    CHECK(op->Setup(bad, ws, ctx) == atb::ERROR_INVALID_TENSOR_INI_MATCH);
    CHECK(atb::DestroyOperation(op) == atb::NO_ERROR);

    atb::infer::ReshapeAndCacheParam rp;
    rp.kvCacheCfg = atb::infer::ReshapeAndCacheParam::K_CACHE_V_CACHE_NZ;
    CHECK(atb::CreateOperation(rp, &op) == atb::ERROR_INVALID_PARAM); // fractal layout of another SoC
    rp.kvCacheCfg = atb::infer::ReshapeAndCacheParam::K_CACHE_V_BYPASS;
    CHECK(atb::CreateOperation(rp, &op) == atb::NO_ERROR);
    CHECK(op->GetInputNum() == 3 && op->GetOutputNum() == 1);
    CHECK(atb::DestroyOperation(op) == atb::NO_ERROR);
    // the cache-management siblings
    atb::infer::BlockCopyParam bp;
    CHECK(atb::CreateOperation(bp, &op) == atb::NO_ERROR);
    CHECK(op->GetName() == "BlockCopyOperation" && op->GetInputNum() == 5 && op->GetOutputNum() == 0);
    CHECK(atb::DestroyOperation(op) == atb::NO_ERROR);
    bp.rsv[0] = 1;
    CHECK(atb::CreateOperation(bp, &op) == atb::ERROR_INVALID_PARAM);
    atb::infer::PagedCacheLoadParam lp;
    CHECK(atb::CreateOperation(lp, &op) == atb::ERROR_INVALID_PARAM); // default = the NZ layout of another SoC
    lp.kvCacheCfg = atb::infer::PagedCacheLoadParam::K_CACHE_V_CACHE_ND;
    lp.isSeqLensCumsumMode = true;
    CHECK(atb::CreateOperation(lp, &op) == atb::NO_ERROR);
    CHECK(op->GetName() == "PagedCacheLoadOperation" && op->GetInputNum() == 7 && op->GetOutputNum() == 2);
    CHECK(atb::DestroyOperation(op) == atb::NO_ERROR);
    atb::infer::KvCacheParam kp;
    CHECK(atb::CreateOperation(kp, &op) == atb::NO_ERROR);
    CHECK(op->GetName() == "KvCacheOperation" && op->GetInputNum() == 5 && op->GetOutputNum() == 0);
    CHECK(atb::DestroyOperation(op) == atb::NO_ERROR);
    // MLA decode attention over the split latent / rope cache
    atb::infer::MultiLatentAttentionParam mp;
    mp.headNum = 128;
    mp.kvHeadNum = 1;
    mp.qkScale = 0.0417f;
    CHECK(atb::CreateOperation(mp, &op) == atb::ERROR_INVALID_PARAM); // default cacheMode KVCACHE has no kernel
    mp.cacheMode = atb::infer::MultiLatentAttentionParam::KROPE_CTKV;
    CHECK(atb::CreateOperation(mp, &op) == atb::NO_ERROR);
    CHECK(op->GetName() == "MultiLatentAttentionOperation" && op->GetInputNum() == 6 && op->GetOutputNum() == 1);
    CHECK(atb::DestroyOperation(op) == atb::NO_ERROR);
    CHECK(atb::DestroyContext(ctx) == atb::NO_ERROR);

    atb::SVector<int> v;
    for (int i = 0; i < 100; ++i) {
        v.push_back(i); // grows past the inline capacity of 64
    }
    CHECK(v.size() == 100 && v.at(99) == 99);
    bool threw = false;
    try {
        v.at(100);
    } catch (const std::out_of_range &) {
        threw = true;
    }
    CHECK(threw);
    std::printf("cpu checks passed\n");
    return 0;
}

static int RunGpu()
{
    const int B = 3, H = 8, HKV = 2, D = 128, BS = 128, NB = 12, MAXB = 3;
    const int32_t lens[B] = {1, 130, 300};
    std::mt19937 rng(7);
    std::normal_distribution<float> nd(0.f, 1.f);
    std::vector<__half> q(B * H * D), kc((size_t)NB * BS * HKV * D), vc(kc.size()), newk(B * HKV * D), newv(B * HKV * D);
    for (auto &x : q) x = __float2half(nd(rng));
    for (auto &x : kc) x = __float2half(nd(rng));
    for (auto &x : vc) x = __float2half(nd(rng));
    for (auto &x : newk) x = __float2half(nd(rng));
    for (auto &x : newv) x = __float2half(nd(rng));
    std::vector<int32_t> bt(B * MAXB, -1), slots(B);
    int next = 0;
    const int perm[NB] = {7, 2, 9, 0, 11, 4, 1, 8, 3, 10, 5, 6};
    for (int b = 0; b < B; ++b) {
        for (int j = 0; j < (lens[b] + BS - 1) / BS; ++j) {
            bt[b * MAXB + j] = perm[next++];
        }
        slots[b] = bt[b * MAXB + (lens[b] - 1) / BS] * BS + (lens[b] - 1) % BS;
    }
    __half *dq, *dk, *dv, *dnk, *dnv, *dout;
    int32_t *dbt, *dlens, *dslots;
    cudaMalloc(&dq, q.size() * 2);
    cudaMalloc(&dk, kc.size() * 2);
    cudaMalloc(&dv, vc.size() * 2);
    cudaMalloc(&dnk, newk.size() * 2);
    cudaMalloc(&dnv, newv.size() * 2);
    cudaMalloc(&dout, q.size() * 2);
    cudaMalloc(&dbt, bt.size() * 4);
    cudaMalloc(&dlens, B * 4);
    cudaMalloc(&dslots, B * 4);
    cudaMemcpy(dq, q.data(), q.size() * 2, cudaMemcpyHostToDevice);
    cudaMemcpy(dk, kc.data(), kc.size() * 2, cudaMemcpyHostToDevice);
    cudaMemcpy(dv, vc.data(), vc.size() * 2, cudaMemcpyHostToDevice);
    cudaMemcpy(dnk, newk.data(), newk.size() * 2, cudaMemcpyHostToDevice);
    cudaMemcpy(dnv, newv.data(), newv.size() * 2, cudaMemcpyHostToDevice);
    cudaMemcpy(dbt, bt.data(), bt.size() * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(dlens, lens, B * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(dslots, slots.data(), B * 4, cudaMemcpyHostToDevice);
    cudaMemset(dout, 0, q.size() * 2);

    cudaStream_t stream;
    CHECK(cudaStreamCreate(&stream) == cudaSuccess);
    atb::Context *ctx = nullptr;
    CHECK(atb::CreateContext(&ctx) == atb::NO_ERROR);
    CHECK(ctx->SetExecuteStream(stream) == atb::NO_ERROR);

    // ---- ReshapeAndCache: outputs alias the caches
    atb::Operation *rac = nullptr;
    CHECK(atb::CreateOperation(atb::infer::ReshapeAndCacheParam{}, &rac) == atb::NO_ERROR);
    atb::VariantPack rp;
    rp.inTensors = {MakeTensor(ACL_FLOAT16, {B, HKV, D}, dnk), MakeTensor(ACL_FLOAT16, {B, HKV, D}, dnv),
                    MakeTensor(ACL_FLOAT16, {NB, BS, HKV, D}, dk), MakeTensor(ACL_FLOAT16, {NB, BS, HKV, D}, dv),
                    MakeTensor(ACL_INT32, {B}, dslots)};
    rp.outTensors = {rp.inTensors.at(2), rp.inTensors.at(3)};
    uint64_t ws = 0;
    CHECK(rac->Setup(rp, ws, ctx) == atb::NO_ERROR && ws == 0);
    CHECK(rac->Execute(rp, nullptr, 0, ctx) == atb::NO_ERROR);
    for (int b = 0; b < B; ++b) { // the same update on the host copy
        std::memcpy(&kc[(size_t)slots[b] * HKV * D], &newk[(size_t)b * HKV * D], HKV * D * 2);
        std::memcpy(&vc[(size_t)slots[b] * HKV * D], &newv[(size_t)b * HKV * D], HKV * D * 2);
    }

    // ---- PagedAttention
    atb::infer::PagedAttentionParam pp;
    pp.headNum = H;
    pp.kvHeadNum = HKV;
    pp.qkScale = 1.f / std::sqrt((float)D);
    atb::Operation *pa = nullptr;
    CHECK(atb::CreateOperation(pp, &pa) == atb::NO_ERROR);
    atb::VariantPack vp;
    vp.inTensors = {MakeTensor(ACL_FLOAT16, {B, H, D}, dq), MakeTensor(ACL_FLOAT16, {NB, BS, HKV, D}, dk),
                    MakeTensor(ACL_FLOAT16, {NB, BS, HKV, D}, dv), MakeTensor(ACL_INT32, {B, MAXB}, dbt),
                    MakeTensor(ACL_INT32, {B}, dlens, const_cast<int32_t *>(lens))};
    vp.outTensors = {MakeTensor(ACL_FLOAT16, {B, H, D}, dout)};
    CHECK(pa->Setup(vp, ws, ctx) == atb::NO_ERROR);
    uint8_t *workspace = nullptr;
    CHECK(cudaMalloc(&workspace, ws) == cudaSuccess);
    CHECK(pa->Execute(vp, workspace, ws - 1, ctx) == atb::ERROR_INVALID_PARAM); // too small a workspace
    CHECK(pa->Execute(vp, workspace, ws, ctx) == atb::NO_ERROR);
    CHECK(cudaStreamSynchronize(stream) == cudaSuccess);

    std::vector<__half> out(q.size()), kback(kc.size());
    cudaMemcpy(out.data(), dout, out.size() * 2, cudaMemcpyDeviceToHost);
    cudaMemcpy(kback.data(), dk, kback.size() * 2, cudaMemcpyDeviceToHost);
    CHECK(std::memcmp(kback.data(), kc.data(), kc.size() * 2) == 0); // ReshapeAndCache is bit-exact

    double max_err = 0;
    for (int b = 0; b < B; ++b) {
        for (int h = 0; h < H; ++h) {
            const int hk = h / (H / HKV);
            std::vector<double> s(lens[b]);
            double m = -1e30;
            for (int t = 0; t < lens[b]; ++t) {
                const size_t row = ((size_t)bt[b * MAXB + t / BS] * BS + t % BS) * HKV + hk;
                double acc = 0;
                for (int d = 0; d < D; ++d) {
                    acc += (double)__half2float(q[(b * H + h) * D + d]) * (double)__half2float(kc[row * D + d]);
                }
                s[t] = acc * pp.qkScale;
                m = std::max(m, s[t]);
            }
            double sum = 0;
            for (auto &x : s) {
                x = std::exp(x - m);
                sum += x;
            }
            for (int d = 0; d < D; ++d) {
                double o = 0;
                for (int t = 0; t < lens[b]; ++t) {
                    const size_t row = ((size_t)bt[b * MAXB + t / BS] * BS + t % BS) * HKV + hk;
                    o += s[t] / sum * (double)__half2float(vc[row * D + d]);
                }
                max_err = std::max(max_err, std::fabs(o - (double)__half2float(out[(b * H + h) * D + d])));
            }
        }
    }
    std::printf("max abs error vs double-precision host attention: %.3e\n", max_err);
    CHECK(max_err <= 4e-3); // 2e-3 vs the golden plus the golden's own rounding of P to fp16
    atb::DestroyOperation(pa);
    atb::DestroyOperation(rac);
    atb::DestroyContext(ctx);
    std::printf("gpu checks passed\n");
    return 0;
}

int main(int argc, char **argv)
{
    if (argc > 1 && std::strcmp(argv[1], "gpu") == 0) {
        return RunGpu();
    }
    return RunCpu();
}
