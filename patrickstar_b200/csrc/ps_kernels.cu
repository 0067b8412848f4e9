// B200 (sm_100a) kernels and C ABI of the chunk optimizer step.
//
// The arithmetic follows the reference's CPU Adam lane by lane
// (patrickstar/ops/csrc/adam/cpu_adam.cpp:33-144): every step is one correctly
// rounded IEEE binary32 operation, spelled with the round-to-nearest
// intrinsics so that nvcc neither fuses nor reorders anything.  The file must
// be compiled without --use_fast_math (no flush-to-zero, precise division and
// square root).
//
// All kernels are streaming and HBM-bound: 128-bit coalesced loads and stores
// with evict-first hints, several independent loads in flight per thread,
// grids sized from the SM count.  There is no contraction, hence no tensor
// core work.
#include "ps_b200.h"

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <memory>
#include <mutex>
#include <new>
#include <unordered_map>

namespace {

constexpr int kThreads = 256;
constexpr int kVec = 8;  // elements per 128-bit fp16 load

thread_local int g_last_cuda_error = 0;
std::atomic<uint64_t> g_launches{0};

// ---------------------------------------------------------------------------
// tuning knobs (ps_tune)
// ---------------------------------------------------------------------------
struct Tuning {
    int unroll = 2;        // 128-bit groups per thread per tile (1, 2 or 4)
    int blocks_per_sm = 0; // 0 = as many as the occupancy calculator allows
    int scan_unroll = 4;
    int bulk = 0;          // 2..4: chunk step with bulk-async (TMA 1-D) staging, that many stages deep
    int fused_depth = 4;   // reduced-gradient loads in flight per thread of the fused multi-GPU step
    int fused_blocks_per_sm = 0;
    int pull_blocks_per_sm = 2;    // staged form of the fused step: grid of the gradient puller
    int staged_blocks_per_sm = 1;  // ... and of the step kernel that runs beside it
    int p2p_unroll = 0;    // 0 = chosen from the world size
    int p2p_blocks_per_sm = 0;
    int fused_min_blocks = 2;  // resident CTAs per SM the fused kernels' register budget is cut for
    int p2p_min_blocks = 2;
};
Tuning g_tune;

#define PS_CUDA(call)                              \
    do {                                           \
        cudaError_t e__ = (call);                  \
        if (e__ != cudaSuccess) {                  \
            g_last_cuda_error = (int)e__;          \
            cudaGetLastError();                    \
            return PS_ERR_CUDA;                    \
        }                                          \
    } while (0)

inline int after_launch()
{
    g_launches.fetch_add(1, std::memory_order_relaxed);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        g_last_cuda_error = (int)e;
        return PS_ERR_CUDA;
    }
    return PS_OK;
}

struct DeviceInfo {
    int device = -1;
    int sm_count = 0;
};

int device_info(DeviceInfo* out)
{
    static std::mutex mu;
    static std::unordered_map<int, int> sm_by_device;
    int dev = 0;
    PS_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(mu);
    auto it = sm_by_device.find(dev);
    if (it == sm_by_device.end()) {
        int sms = 0;
        PS_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        it = sm_by_device.emplace(dev, sms).first;
    }
    out->device = dev;
    out->sm_count = it->second;
    return PS_OK;
}

// ---------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------
struct Slot {
    float loss_scale, beta1, beta2, b1m1, b2m1, bias2_sqrt, eps, step_size, wd, w_decay, clip,
        divisor;
    int adamw;
    float inv_scale;  // 1 / loss_scale when that is exact (power-of-two scale), else 0
    float inv_div;    // float(1 / divisor): the factor torch multiplies with for `payload /= world`
};

__device__ __forceinline__ Slot load_slot(const ps_hyper_slot* s)
{
    // plain loads: the slot lives in global memory (chunk-level kernel) or in
    // shared memory (tensor-level kernel)
    const uint4* q = reinterpret_cast<const uint4*>(s);
    uint4 a = q[0], b = q[1], c = q[2], d = q[3];
    Slot r;
    r.loss_scale = __uint_as_float(a.x);
    r.beta1 = __uint_as_float(a.y);
    r.beta2 = __uint_as_float(a.z);
    r.b1m1 = __uint_as_float(a.w);
    r.b2m1 = __uint_as_float(b.x);
    r.bias2_sqrt = __uint_as_float(b.y);
    r.eps = __uint_as_float(b.z);
    r.step_size = __uint_as_float(b.w);
    r.wd = __uint_as_float(c.x);
    r.w_decay = __uint_as_float(c.y);
    r.clip = __uint_as_float(c.z);
    r.divisor = __uint_as_float(c.w);
    r.adamw = (int)d.x;
    r.inv_scale = __uint_as_float(d.y);
    r.inv_div = __uint_as_float(d.z);
    return r;
}

__device__ __forceinline__ Slot slot_from_value(const ps_hyper_slot& s)
{
    Slot r;
    r.loss_scale = s.loss_scale;
    r.beta1 = s.beta1;
    r.beta2 = s.beta2;
    r.b1m1 = s.beta1_minus1;
    r.b2m1 = s.beta2_minus1;
    r.bias2_sqrt = s.bias2_sqrt;
    r.eps = s.eps;
    r.step_size = s.step_size;
    r.wd = s.weight_decay;
    r.w_decay = s.w_decay;
    r.clip = s.clip;
    r.divisor = s.grad_divisor;
    r.adamw = s.adamw_mode;
    r.inv_scale = s.inv_loss_scale;
    r.inv_div = s.inv_grad_divisor;
    return r;
}

__device__ __forceinline__ float half_bits_to_float(uint32_t h)
{
    return __half2float(__ushort_as_half((unsigned short)h));
}
__device__ __forceinline__ uint32_t float_to_half_bits(float f)
{
    return (uint32_t)__half_as_ushort(__float2half_rn(f));
}

// clamp_(-c, c) as torch does it: a NaN stays a NaN (fminf / fmaxf alone would
// turn it into -c and hide a diverged gradient when no overflow gate is active).
__device__ __forceinline__ float clamp_keep_nan(float g, float c)
{
    return g != g ? g : fminf(fmaxf(g, -c), c);
}

// fp16 gradient as the step sees it: the fp16 `payload /= world_size` of
// patrickstar/core/client.py:838 and the fp16 clamp_ of
// patrickstar/ops/fp16_cpu_adam.py:365-379, each rounded back to fp16.
// The division of a CUDA fp16 tensor by a Python scalar is computed by torch as
// half(float(g) * (1.0f / world)); for a power-of-two world that equals the true
// quotient, for any other it can differ from it by one fp16 ulp.
__device__ __forceinline__ float grad_from_half(uint32_t h, const Slot& s)
{
    float g = half_bits_to_float(h);
    if (s.divisor > 1.f) {
        const float inv = s.inv_div != 0.f ? s.inv_div : __fdiv_rn(1.0f, s.divisor);
        g = half_bits_to_float(float_to_half_bits(__fmul_rn(g, inv)));
    }
    if (s.clip > 0.f) g = half_bits_to_float(float_to_half_bits(clamp_keep_nan(g, s.clip)));
    return g;
}

// 1 / scale when scale is a positive power of two whose reciprocal is a normal float, else 0.
__host__ __device__ __forceinline__ float exact_reciprocal_or_zero(float scale)
{
    union { float f; uint32_t u; } a, r;
    a.f = scale;
    const uint32_t e = (a.u >> 23) & 0xffu;
    if ((a.u & 0x807fffffu) != 0u || e == 0u || e > 253u) return 0.f;
    r.u = (254u - e) << 23;
    return r.f;
}

// One element of Adam_Optimizer::Step's SIMD body (cpu_adam.cpp:91-143).
__device__ __forceinline__ void adam_element(float g, float& p, float& m, float& v, const Slot& s)
{
    // g / scale.  For a power-of-two scale the product with the exact reciprocal is the same
    // correctly rounded value (both round the same real number), and costs one instruction
    // instead of a division sequence.
    if (s.inv_scale != 0.f)
        g = __fmul_rn(g, s.inv_scale);
    else if (s.loss_scale > 0.f)
        g = __fdiv_rn(g, s.loss_scale);
    if (s.wd > 0.f && !s.adamw) g = __fmaf_rn(p, s.wd, g);
    m = __fmul_rn(m, s.beta1);
    m = __fmaf_rn(g, s.b1m1, m);
    v = __fmul_rn(v, s.beta2);
    g = __fmul_rn(g, g);
    v = __fmaf_rn(g, s.b2m1, v);
    g = __fsqrt_rn(v);
    g = __fmaf_rn(g, s.bias2_sqrt, s.eps);
    g = __fdiv_rn(m, g);
    if (s.wd > 0.f && s.adamw) p = __fmaf_rn(p, s.w_decay, p);
    p = __fmaf_rn(g, s.step_size, p);
}

__device__ __forceinline__ uint4 ld_stream(const uint4* p) { return __ldcs(p); }
__device__ __forceinline__ float4 ld_stream(const float4* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(uint4* p, uint4 v) { __stcs(p, v); }
__device__ __forceinline__ void st_stream(float4* p, float4 v) { __stcs(p, v); }

// NVSwitch multicast ("multimem") accesses on an address of the fp16 chunk
// buffer's multicast mapping: the load returns the SUM over every rank's copy
// (added in the switch, accumulated in fp32, rounded once to fp16), the store
// writes every rank's copy.  They fuse the reduce-scatter of the gradient
// chunks and the all-gather of the param chunks into the step kernel.
__device__ __forceinline__ uint4 mm_ld_reduce_f16x8(const void* mc)
{
    uint4 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(mc)
                 : "memory");
    return r;
}
__device__ __forceinline__ void mm_st_f16x8(void* mc, uint4 v)
{
    asm volatile("multimem.st.relaxed.sys.global.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x),
                 "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}
// One element: there is no 16-bit multimem access, so a single gradient is taken
// out of the reduced f16x2 pair that holds it (the two lanes are summed
// independently), and a single fp16 param is stored to every rank's buffer with
// plain peer stores.
struct McCtx {
    long long mc_delta;                 // multicast mapping minus local fp16 buffer, in bytes
    const unsigned long long* peers;    // every rank's fp16 buffer base (device array): where params are stored
    const unsigned long long* gather;   // per rank, where its gradients are read from: the same bases
                                        // (peer loads), or local staging copies biased by the chunk's offset
    const char* local_base;             // this rank's fp16 buffer base
    int world;
};
__device__ __forceinline__ uint32_t mm_ld_reduce_f16(const uint16_t* local_elem, const McCtx& mc)
{
    const uintptr_t a = reinterpret_cast<uintptr_t>(local_elem);
    const char* pair = reinterpret_cast<const char*>(a & ~(uintptr_t)3) + mc.mc_delta;
    uint32_t r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.f16x2 %0, [%1];"
                 : "=r"(r)
                 : "l"(pair)
                 : "memory");
    return (a & 2) ? (r >> 16) : (r & 0xffffu);
}
__device__ __forceinline__ void peers_st_f16(uint16_t* local_elem, uint32_t h, const McCtx& mc)
{
    const long long off = reinterpret_cast<const char*>(local_elem) - mc.local_base;
    for (int r = 0; r < mc.world; ++r)
        *reinterpret_cast<uint16_t*>(mc.peers[r] + off) = (uint16_t)h;
}

// Peer-to-peer form of the same fusion, over plain peer mappings of every
// rank's fp16 buffer: the gradient of an element is the sum of the W ranks'
// values, accumulated in fp32 in rank order and rounded once to fp16; the
// updated param is stored into every rank's buffer.
constexpr int kMaxPeers = 8;
// kColl values of the step templates: 0 no collective, 1 multimem, 2 / 24 / 22
// peer-to-peer compiled for up to 8 / 4 / 2 ranks (fewer ranks, fewer registers),
// 38 / 34 / 32 the same summation over copies that the copy engines have brought
// into local staging buffers, with the params stored locally only
__host__ __device__ constexpr int peers_of(int kColl)
{
    return (kColl == 22 || kColl == 32) ? 2 : ((kColl == 24 || kColl == 34) ? 4 : 8);
}
__host__ __device__ constexpr bool is_staged_copies(int kColl) { return kColl == 32 || kColl == 34 || kColl == 38; }
__host__ __device__ constexpr bool is_p2p(int kColl)
{
    return kColl == 2 || kColl == 22 || kColl == 24 || is_staged_copies(kColl);
}

template <int NP>
__device__ __forceinline__ uint4 p2p_ld_reduce_f16x8(const uint16_t* local_vec, const McCtx& mc)
{
    const long long off = reinterpret_cast<const char*>(local_vec) - mc.local_base;
    uint4 q[NP];
#pragma unroll
    for (int r = 0; r < NP; ++r)
        if (r < mc.world) q[r] = *reinterpret_cast<const uint4*>(mc.gather[r] + off);
    float acc[8];
    uint32_t w0[4] = {q[0].x, q[0].y, q[0].z, q[0].w};
#pragma unroll
    for (int k = 0; k < 8; ++k)
        acc[k] = half_bits_to_float((k & 1) ? (w0[k >> 1] >> 16) : (w0[k >> 1] & 0xffffu));
#pragma unroll
    for (int r = 1; r < NP; ++r) {
        if (r < mc.world) {
            uint32_t w[4] = {q[r].x, q[r].y, q[r].z, q[r].w};
#pragma unroll
            for (int k = 0; k < 8; ++k)
                acc[k] = __fadd_rn(acc[k], half_bits_to_float((k & 1) ? (w[k >> 1] >> 16) : (w[k >> 1] & 0xffffu)));
        }
    }
    uint4 out;
    out.x = float_to_half_bits(acc[0]) | (float_to_half_bits(acc[1]) << 16);
    out.y = float_to_half_bits(acc[2]) | (float_to_half_bits(acc[3]) << 16);
    out.z = float_to_half_bits(acc[4]) | (float_to_half_bits(acc[5]) << 16);
    out.w = float_to_half_bits(acc[6]) | (float_to_half_bits(acc[7]) << 16);
    return out;
}
__device__ __forceinline__ uint32_t p2p_ld_reduce_f16(const uint16_t* local_elem, const McCtx& mc)
{
    const long long off = reinterpret_cast<const char*>(local_elem) - mc.local_base;
    float acc = half_bits_to_float(*reinterpret_cast<const uint16_t*>(mc.gather[0] + off));
    for (int r = 1; r < mc.world; ++r)
        acc = __fadd_rn(acc, half_bits_to_float(*reinterpret_cast<const uint16_t*>(mc.gather[r] + off)));
    return float_to_half_bits(acc);
}
template <int NP>
__device__ __forceinline__ void p2p_st_f16x8(uint16_t* local_vec, uint4 v, const McCtx& mc)
{
    const long long off = reinterpret_cast<const char*>(local_vec) - mc.local_base;
#pragma unroll
    for (int r = 0; r < NP; ++r)
        if (r < mc.world) *reinterpret_cast<uint4*>(mc.peers[r] + off) = v;
}

// Index (absolute, in the segment table) of the last segment of [lo, hi) whose
// start is <= e; lo when none starts at or before e.
__device__ __forceinline__ uint32_t find_segment(const ps_segment* segs, uint32_t lo, uint32_t hi,
                                                 uint32_t e)
{
    uint32_t a = lo, b = hi;  // invariant: answer in [a, b)
    while (b - a > 1) {
        uint32_t mid = a + ((b - a) >> 1);
        if (segs[mid].start <= e)
            a = mid;
        else
            b = mid;
    }
    return a;
}

struct SegView {
    uint32_t start, end, slot;
};
__device__ __forceinline__ SegView load_segment(const ps_segment* segs, uint32_t i)
{
    uint4 q = *reinterpret_cast<const uint4*>(segs + i);
    return SegView{q.x, q.y, q.z};
}

// Element-wise path for a group of up to 8 elements that is ragged (chunk end)
// or straddles a segment boundary.  Scalar loads and stores; every element
// looks up its own segment.
template <bool kRestore, bool kGradHalf, int kColl = 0>
__device__ __noinline__ void slow_group(const ps_chunk_desc d, const void* grads,
                                        const ps_segment* segs, uint32_t seg_lo, uint32_t seg_hi,
                                        const ps_hyper_slot* slots, uint32_t e, uint32_t e_end,
                                        uint32_t si, uint16_t* p16_out, McCtx mc = McCtx())
{
    for (uint32_t i = e; i < e_end; ++i) {
        SegView sv = load_segment(segs, si);
        while (i >= sv.end && si + 1 < seg_hi) {
            ++si;
            sv = load_segment(segs, si);
        }
        if (i < sv.start || i >= sv.end) continue;
        float p = d.p32[i];
        if (kRestore) {
            if (kColl && !is_staged_copies(kColl))
                peers_st_f16(p16_out + i, float_to_half_bits(p), mc);
            else if (p16_out)
                p16_out[i] = (uint16_t)float_to_half_bits(p);
            continue;
        }
        Slot s = load_slot(slots + sv.slot);
        float g;
        if (kColl == 1)
            g = grad_from_half(mm_ld_reduce_f16(reinterpret_cast<const uint16_t*>(grads) + i, mc), s);
        else if (is_p2p(kColl))
            g = grad_from_half(p2p_ld_reduce_f16(reinterpret_cast<const uint16_t*>(grads) + i, mc), s);
        else if (kGradHalf)
            g = grad_from_half(reinterpret_cast<const uint16_t*>(grads)[i], s);
        else
            g = reinterpret_cast<const float*>(grads)[i];
        float m = d.exp_avg[i], v = d.exp_avg_sq[i];
        adam_element(g, p, m, v, s);
        d.p32[i] = p;
        d.exp_avg[i] = m;
        d.exp_avg_sq[i] = v;
        if (kColl && !is_staged_copies(kColl))
            peers_st_f16(p16_out + i, float_to_half_bits(p), mc);
        else if (p16_out)
            p16_out[i] = (uint16_t)float_to_half_bits(p);
    }
}

// One tile of one chunk: U groups of 8 elements per thread, group j of thread t
// at tile_base + (j * kThreads + t) * 8, so that every warp-wide access is one
// contiguous 512-byte (fp16) or 2 x 512-byte (fp32) run.  All loads of the tile
// are issued before the first dependent instruction.
template <int U, bool kRestore, bool kWrite16, int kColl = 0, bool kPre = false>
__device__ __forceinline__ void step_tile(const ps_chunk_desc& d, const ps_segment* segs,
                                          const ps_hyper_slot* slots, uint32_t tile_base,
                                          McCtx mc = McCtx(), const uint4* pre = nullptr)
{
    uint4 gq[U];
    float4 pq[U][2], mq[U][2], vq[U][2];
    uint32_t e[U];
    bool full[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
        e[j] = tile_base + (uint32_t)(j * kThreads + threadIdx.x) * kVec;
        full[j] = (e[j] + kVec <= d.numel);
        if (full[j]) {
            const float4* pp = reinterpret_cast<const float4*>(d.p32 + e[j]);
            pq[j][0] = ld_stream(pp);
            pq[j][1] = ld_stream(pp + 1);
            if (!kRestore) {
                if (kPre)
                    gq[j] = pre[j];  // loaded by the caller some tiles ago
                else if (kColl == 1)
                    gq[j] = mm_ld_reduce_f16x8(reinterpret_cast<const char*>(d.h16 + e[j]) + mc.mc_delta);
                else if (is_p2p(kColl))
                    gq[j] = p2p_ld_reduce_f16x8<peers_of(kColl)>(d.h16 + e[j], mc);
                else
                    gq[j] = ld_stream(reinterpret_cast<const uint4*>(d.h16 + e[j]));
                const float4* mp = reinterpret_cast<const float4*>(d.exp_avg + e[j]);
                const float4* vp = reinterpret_cast<const float4*>(d.exp_avg_sq + e[j]);
                mq[j][0] = ld_stream(mp);
                mq[j][1] = ld_stream(mp + 1);
                vq[j][0] = ld_stream(vp);
                vq[j][1] = ld_stream(vp + 1);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < U; ++j) {
        if (e[j] >= d.numel) continue;
        uint32_t si = d.seg_begin;
        if (d.seg_end - d.seg_begin > 1) si = find_segment(segs, d.seg_begin, d.seg_end, e[j]);
        SegView sv = load_segment(segs, si);
        if (!(full[j] && sv.start <= e[j] && e[j] + kVec <= sv.end)) {
            uint32_t e_end = e[j] + kVec < d.numel ? e[j] + kVec : d.numel;
            slow_group<kRestore, true, kColl>(d, d.h16, segs, d.seg_begin, d.seg_end, slots, e[j], e_end,
                                            si, kWrite16 ? d.h16 : nullptr, mc);
            continue;
        }
        float p[8] = {pq[j][0].x, pq[j][0].y, pq[j][0].z, pq[j][0].w,
                      pq[j][1].x, pq[j][1].y, pq[j][1].z, pq[j][1].w};
        if (!kRestore) {
            Slot s = load_slot(slots + sv.slot);
            float m[8] = {mq[j][0].x, mq[j][0].y, mq[j][0].z, mq[j][0].w,
                          mq[j][1].x, mq[j][1].y, mq[j][1].z, mq[j][1].w};
            float v[8] = {vq[j][0].x, vq[j][0].y, vq[j][0].z, vq[j][0].w,
                          vq[j][1].x, vq[j][1].y, vq[j][1].z, vq[j][1].w};
            uint32_t gw[4] = {gq[j].x, gq[j].y, gq[j].z, gq[j].w};
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                uint32_t h = (k & 1) ? (gw[k >> 1] >> 16) : (gw[k >> 1] & 0xffffu);
                adam_element(grad_from_half(h, s), p[k], m[k], v[k], s);
            }
            float4* pp = reinterpret_cast<float4*>(d.p32 + e[j]);
            float4* mp = reinterpret_cast<float4*>(d.exp_avg + e[j]);
            float4* vp = reinterpret_cast<float4*>(d.exp_avg_sq + e[j]);
            st_stream(pp, make_float4(p[0], p[1], p[2], p[3]));
            st_stream(pp + 1, make_float4(p[4], p[5], p[6], p[7]));
            st_stream(mp, make_float4(m[0], m[1], m[2], m[3]));
            st_stream(mp + 1, make_float4(m[4], m[5], m[6], m[7]));
            st_stream(vp, make_float4(v[0], v[1], v[2], v[3]));
            st_stream(vp + 1, make_float4(v[4], v[5], v[6], v[7]));
        }
        if (!kWrite16) continue;
        uint4 out;
        out.x = float_to_half_bits(p[0]) | (float_to_half_bits(p[1]) << 16);
        out.y = float_to_half_bits(p[2]) | (float_to_half_bits(p[3]) << 16);
        out.z = float_to_half_bits(p[4]) | (float_to_half_bits(p[5]) << 16);
        out.w = float_to_half_bits(p[6]) | (float_to_half_bits(p[7]) << 16);
        if (kColl == 1)
            mm_st_f16x8(reinterpret_cast<char*>(d.h16 + e[j]) + mc.mc_delta, out);
        else if (is_p2p(kColl) && !is_staged_copies(kColl))
            p2p_st_f16x8<peers_of(kColl)>(d.h16 + e[j], out, mc);
        else
            st_stream(reinterpret_cast<uint4*>(d.h16 + e[j]), out);
    }
}

__device__ __forceinline__ ps_chunk_desc load_desc(const ps_chunk_desc* c)
{
    const uint4* q = reinterpret_cast<const uint4*>(c);
    uint4 a = __ldg(q), b = __ldg(q + 1), w = __ldg(q + 2);
    ps_chunk_desc d;
    d.p32 = reinterpret_cast<float*>(((unsigned long long)a.y << 32) | a.x);
    d.exp_avg = reinterpret_cast<float*>(((unsigned long long)a.w << 32) | a.z);
    d.exp_avg_sq = reinterpret_cast<float*>(((unsigned long long)b.y << 32) | b.x);
    d.h16 = reinterpret_cast<uint16_t*>(((unsigned long long)b.w << 32) | b.z);
    d.numel = w.x;
    d.seg_begin = w.y;
    d.seg_end = w.z;
    d.reserved = w.w;
    return d;
}

// The fused chunk step over a table of chunks.  Tiles are numbered chunk-major;
// consecutive CTAs take consecutive tiles, then stride by the grid.
template <int U>
__global__ void __launch_bounds__(kThreads)
chunk_step_kernel(const ps_chunk_desc* __restrict__ chunks, uint32_t n_chunks,
                  uint32_t tiles_per_chunk, const ps_segment* __restrict__ segs,
                  const ps_step_ctrl* __restrict__ ctrl)
{
    constexpr uint32_t kTile = kThreads * kVec * U;
    const int skip = __ldg(&ctrl->skip);
    const ps_hyper_slot* slots = ctrl->slots;
    const uint64_t total = (uint64_t)n_chunks * tiles_per_chunk;
    for (uint64_t t = blockIdx.x; t < total; t += gridDim.x) {
        const uint32_t c = (uint32_t)(t / tiles_per_chunk);
        const uint32_t lt = (uint32_t)(t - (uint64_t)c * tiles_per_chunk);
        const ps_chunk_desc d = load_desc(chunks + c);
        const uint32_t tile_base = d.reserved + lt * kTile;  // d.reserved = first element (0 for a whole chunk)
        if (tile_base >= d.numel) continue;
        if (skip)
            step_tile<U, true, true>(d, segs, slots, tile_base);
        else
            step_tile<U, false, true>(d, segs, slots, tile_base);
    }
}

// ---------------------------------------------------------------------------
// Chunk step with bulk-async staging: the four input streams of a tile (fp16
// grads, fp32 master / momentum / variance; 28 KB per 2048 elements) are brought
// into shared memory by the copy engine of the SM (cp.async.bulk, completion
// counted on an mbarrier), kBulkStages tiles deep, so the bytes in flight are
// bounded by shared memory and not by registers.  One elected thread issues the
// copies; all threads wait on the stage's barrier, pull their elements out of
// shared memory, hand the stage back, and compute and store from registers.
// Every wait is bounded: on a timeout the CTA records an error bit in the
// control block and leaves.
// ---------------------------------------------------------------------------
constexpr uint32_t kBulkTile = kThreads * kVec;  // 2048 elements
struct __align__(128) BulkStage {
    uint16_t g[kBulkTile];
    float p[kBulkTile];
    float m[kBulkTile];
    float v[kBulkTile];
};
constexpr uint32_t kBulkStageBytes = sizeof(BulkStage);
static_assert(kBulkStageBytes == 28672, "stage layout");

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
// Streaming data: read once, so the copy carries an evict-first L2 policy like
// the ld.global.cs of the register path.
__device__ __forceinline__ uint64_t l2_evict_first_policy()
{
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ void bulk_load(void* dst_smem, const void* src, uint32_t bytes, uint64_t* bar,
                                          uint64_t policy)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            smem_u32(dst_smem)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
// Bounded wait for the phase with the given parity.  False = gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity)
{
    const uint32_t addr = smem_u32(bar);
    for (uint32_t spin = 0; spin < (1u << 26); ++spin) {
        uint32_t done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

// Four consecutive elements of one thread, data already in registers.
__device__ __forceinline__ void adam_group4(const ps_chunk_desc& d, const ps_segment* segs,
                                            const ps_hyper_slot* slots, uint32_t e, uint2 gq, float4 pq,
                                            float4 mq, float4 vq)
{
    uint32_t si = d.seg_begin;
    if (d.seg_end - d.seg_begin > 1) si = find_segment(segs, d.seg_begin, d.seg_end, e);
    const SegView sv = load_segment(segs, si);
    if (!(sv.start <= e && e + 4 <= sv.end)) {
        slow_group<false, true>(d, d.h16, segs, d.seg_begin, d.seg_end, slots, e, e + 4, si, d.h16);
        return;
    }
    const Slot s = load_slot(slots + sv.slot);
    float p[4] = {pq.x, pq.y, pq.z, pq.w};
    float m[4] = {mq.x, mq.y, mq.z, mq.w};
    float v[4] = {vq.x, vq.y, vq.z, vq.w};
    const uint32_t gw[2] = {gq.x, gq.y};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t h = (k & 1) ? (gw[k >> 1] >> 16) : (gw[k >> 1] & 0xffffu);
        adam_element(grad_from_half(h, s), p[k], m[k], v[k], s);
    }
    __stcs(reinterpret_cast<float4*>(d.p32 + e), make_float4(p[0], p[1], p[2], p[3]));
    __stcs(reinterpret_cast<float4*>(d.exp_avg + e), make_float4(m[0], m[1], m[2], m[3]));
    __stcs(reinterpret_cast<float4*>(d.exp_avg_sq + e), make_float4(v[0], v[1], v[2], v[3]));
    uint2 out;
    out.x = float_to_half_bits(p[0]) | (float_to_half_bits(p[1]) << 16);
    out.y = float_to_half_bits(p[2]) | (float_to_half_bits(p[3]) << 16);
    __stcs(reinterpret_cast<uint2*>(d.h16 + e), out);
}

template <int kBulkStages>
__global__ void __launch_bounds__(kThreads)
chunk_step_bulk_kernel(const ps_chunk_desc* __restrict__ chunks, uint32_t n_chunks,
                       uint32_t tiles_per_chunk, const ps_segment* __restrict__ segs,
                       const ps_step_ctrl* __restrict__ ctrl)
{
    extern __shared__ __align__(128) unsigned char bulk_smem[];
    BulkStage* stages = reinterpret_cast<BulkStage*>(bulk_smem);
    __shared__ uint64_t full_bar[kBulkStages];
    const ps_hyper_slot* slots = ctrl->slots;
    const uint64_t total = (uint64_t)n_chunks * tiles_per_chunk;
    const uint64_t stride = gridDim.x;
    if (__ldg(&ctrl->skip)) {
        // restore path: plain loads, no staging needed (6 B per element)
        for (uint64_t t = blockIdx.x; t < total; t += stride) {
            const uint32_t c = (uint32_t)(t / tiles_per_chunk);
            const uint32_t lt = (uint32_t)(t - (uint64_t)c * tiles_per_chunk);
            const ps_chunk_desc d = load_desc(chunks + c);
            const uint32_t tile_base = d.reserved + lt * kBulkTile;
            if (tile_base < d.numel) step_tile<1, true, true>(d, segs, slots, tile_base);
        }
        return;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < kBulkStages; ++s) mbar_init(&full_bar[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // producer cursor (thread 0 only): next position of this CTA's tile sequence to look at,
    // and the number of staged tiles issued so far
    uint64_t prod_t = blockIdx.x;
    uint32_t prod_n = 0;
    const uint64_t policy = l2_evict_first_policy();
    auto issue_next = [&]() {
        while (prod_t < total) {
            const uint32_t c = (uint32_t)(prod_t / tiles_per_chunk);
            const uint32_t lt = (uint32_t)(prod_t - (uint64_t)c * tiles_per_chunk);
            const ps_chunk_desc d = load_desc(chunks + c);
            const uint32_t tile_base = d.reserved + lt * kBulkTile;
            prod_t += stride;
            if (tile_base + kBulkTile <= d.numel) {  // a full tile: staged
                BulkStage* st = &stages[prod_n % kBulkStages];
                uint64_t* bar = &full_bar[prod_n % kBulkStages];
                mbar_expect_tx(bar, kBulkStageBytes);
                bulk_load(st->g, d.h16 + tile_base, sizeof(st->g), bar, policy);
                bulk_load(st->p, d.p32 + tile_base, sizeof(st->p), bar, policy);
                bulk_load(st->m, d.exp_avg + tile_base, sizeof(st->m), bar, policy);
                bulk_load(st->v, d.exp_avg_sq + tile_base, sizeof(st->v), bar, policy);
                ++prod_n;
                return;
            }
        }
    };
    if (threadIdx.x == 0)
        for (int s = 0; s < kBulkStages; ++s) issue_next();

    uint32_t cons_n = 0;
    for (uint64_t t = blockIdx.x; t < total; t += stride) {
        const uint32_t c = (uint32_t)(t / tiles_per_chunk);
        const uint32_t lt = (uint32_t)(t - (uint64_t)c * tiles_per_chunk);
        const ps_chunk_desc d = load_desc(chunks + c);
        const uint32_t tile_base = d.reserved + lt * kBulkTile;
        if (tile_base >= d.numel) continue;
        if (tile_base + kBulkTile > d.numel) {  // ragged last tile of a chunk: plain path
            step_tile<1, false, true>(d, segs, slots, tile_base);
            continue;
        }
        const uint32_t s = cons_n % kBulkStages;
        const bool arrived = mbar_wait(&full_bar[s], (cons_n / kBulkStages) & 1u);
        if (!__syncthreads_and(arrived)) {
            // Gave up on this stage.  Copies of the stages issued after it may still be
            // landing in this CTA's shared memory, which the next resident CTA may own:
            // wait (bounded again) for each of them before leaving.
            if (threadIdx.x == 0) {
                atomicOr(const_cast<int32_t*>(&ctrl->error), 2);
                for (uint32_t i = cons_n; i < prod_n; ++i)
                    mbar_wait(&full_bar[i % kBulkStages], (i / kBulkStages) & 1u);
            }
            __syncthreads();
            return;
        }
        // thread i owns elements [4i, 4i+4) and [1024+4i, 1024+4i+4) of the tile:
        // 16-byte (fp32) and 8-byte (fp16) shared-memory reads with unit stride across the warp
        const BulkStage* st = &stages[s];
        const uint32_t o0 = threadIdx.x * 4, o1 = kBulkTile / 2 + threadIdx.x * 4;
        const uint2 g0 = *reinterpret_cast<const uint2*>(st->g + o0);
        const uint2 g1 = *reinterpret_cast<const uint2*>(st->g + o1);
        const float4 p0 = *reinterpret_cast<const float4*>(st->p + o0);
        const float4 p1 = *reinterpret_cast<const float4*>(st->p + o1);
        const float4 m0 = *reinterpret_cast<const float4*>(st->m + o0);
        const float4 m1 = *reinterpret_cast<const float4*>(st->m + o1);
        const float4 v0 = *reinterpret_cast<const float4*>(st->v + o0);
        const float4 v1 = *reinterpret_cast<const float4*>(st->v + o1);
        __syncthreads();  // the stage has been read by everyone: it may be refilled
        if (threadIdx.x == 0) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue_next();
        }
        ++cons_n;
        adam_group4(d, segs, slots, tile_base + o0, g0, p0, m0, v0);
        adam_group4(d, segs, slots, tile_base + o1, g1, p1, m1, v1);
    }
}

// The chunk step fused with its two collectives (multi-GPU): the gradient of an
// element is the switch-side sum over all ranks' fp16 buffers (the
// reduce-scatter), the updated fp16 param is stored to all ranks' buffers (the
// all-gather).  `mc_delta` is the byte distance from this rank's fp16 buffer to
// its multicast mapping.  Every element is read and then written by the one
// thread that owns it, on the one rank that owns its chunk, so no rank-to-rank
// ordering is needed inside the kernel; the caller brackets the launch with
// barriers across ranks (gradients complete before, params visible after).
//
// The kernel is bound by NVLink, whose round trip through the switch is several
// times the HBM latency, so the reduced gradient loads run kFusedDepth tiles
// ahead of the rest: a thread keeps that many 16-byte multimem loads in flight
// in a register ring while it works on the current tile (one 8-element group
// per thread and tile, to leave the registers to the ring).
__device__ __forceinline__ uint4 fused_prefetch(const ps_chunk_desc* chunks, uint32_t tiles_per_chunk,
                                                uint64_t t, uint64_t total, int skip, const McCtx& mc)
{
    uint4 g = make_uint4(0u, 0u, 0u, 0u);
    if (skip || t >= total) return g;
    const uint32_t c = (uint32_t)(t / tiles_per_chunk);
    const uint32_t lt = (uint32_t)(t - (uint64_t)c * tiles_per_chunk);
    const uint16_t* h16 = reinterpret_cast<const uint16_t*>(
        __ldg(reinterpret_cast<const unsigned long long*>(&chunks[c].h16)));
    const uint32_t numel = __ldg(&chunks[c].numel);
    const uint32_t e = lt * (uint32_t)(kThreads * kVec) + threadIdx.x * kVec;
    if (e + kVec <= numel) g = mm_ld_reduce_f16x8(reinterpret_cast<const char*>(h16 + e) + mc.mc_delta);
    return g;
}

template <int kFusedDepth, int kMinBlocks>
__global__ void __launch_bounds__(kThreads, kMinBlocks)
chunk_step_fused_kernel(const ps_chunk_desc* __restrict__ chunks, uint32_t n_chunks,
                        uint32_t tiles_per_chunk, const ps_segment* __restrict__ segs,
                        const ps_step_ctrl* __restrict__ ctrl, McCtx mc)
{
    constexpr uint32_t kTile = kThreads * kVec;
    const int skip = __ldg(&ctrl->skip);
    const ps_hyper_slot* slots = ctrl->slots;
    const uint64_t total = (uint64_t)n_chunks * tiles_per_chunk;
    const uint64_t stride = gridDim.x;
    uint4 ring[kFusedDepth];
#pragma unroll
    for (int k = 0; k < kFusedDepth; ++k)
        ring[k] = fused_prefetch(chunks, tiles_per_chunk, blockIdx.x + (uint64_t)k * stride, total, skip, mc);
    uint64_t t = blockIdx.x;
    while (t < total) {
#pragma unroll
        for (int k = 0; k < kFusedDepth; ++k) {
            if (t < total) {
                const uint4 g = ring[k];
                ring[k] = fused_prefetch(chunks, tiles_per_chunk, t + (uint64_t)kFusedDepth * stride, total,
                                         skip, mc);
                const uint32_t c = (uint32_t)(t / tiles_per_chunk);
                const uint32_t lt = (uint32_t)(t - (uint64_t)c * tiles_per_chunk);
                const ps_chunk_desc d = load_desc(chunks + c);
                const uint32_t tile_base = lt * kTile;
                if (tile_base < d.numel) {
                    if (skip)
                        step_tile<1, true, true, 1, false>(d, segs, slots, tile_base, mc);
                    else
                        step_tile<1, false, true, 1, true>(d, segs, slots, tile_base, mc, &g);
                }
                t += stride;
            }
        }
    }
    // the params stored to the other ranks are ordered before the end of the kernel
    __threadfence_system();
}

// Peer-to-peer form of the fused kernel (no multicast object needed; the sums are
// exact fp32 accumulations).  Enough independent peer loads are in flight per
// thread (W per 8-element group) that no register ring is needed.
template <int U, int kColl, int kMinBlocks>
__global__ void __launch_bounds__(kThreads, kMinBlocks)
chunk_step_p2p_kernel(const ps_chunk_desc* __restrict__ chunks, uint32_t n_chunks,
                      uint32_t tiles_per_chunk, const ps_segment* __restrict__ segs,
                      const ps_step_ctrl* __restrict__ ctrl, McCtx mc)
{
    constexpr uint32_t kTile = kThreads * kVec * U;
    const int skip = __ldg(&ctrl->skip);
    const ps_hyper_slot* slots = ctrl->slots;
    const uint64_t total = (uint64_t)n_chunks * tiles_per_chunk;
    for (uint64_t t = blockIdx.x; t < total; t += gridDim.x) {
        const uint32_t c = (uint32_t)(t / tiles_per_chunk);
        const uint32_t lt = (uint32_t)(t - (uint64_t)c * tiles_per_chunk);
        const ps_chunk_desc d = load_desc(chunks + c);
        const uint32_t tile_base = lt * kTile;
        if (tile_base >= d.numel) continue;
        if (skip)
            step_tile<U, true, true, kColl>(d, segs, slots, tile_base, mc);
        else
            step_tile<U, false, true, kColl>(d, segs, slots, tile_base, mc);
    }
    __threadfence_system();
}

// Restore alone (fp16_cpu_adam.py:298-309): fp16 slot := half(fp32 master) for every
// segment of every chunk, no control block.
template <int U>
__global__ void __launch_bounds__(kThreads)
chunk_restore_kernel(const ps_chunk_desc* __restrict__ chunks, uint32_t n_chunks,
                     uint32_t tiles_per_chunk, const ps_segment* __restrict__ segs)
{
    constexpr uint32_t kTile = kThreads * kVec * U;
    const uint64_t total = (uint64_t)n_chunks * tiles_per_chunk;
    for (uint64_t t = blockIdx.x; t < total; t += gridDim.x) {
        const uint32_t c = (uint32_t)(t / tiles_per_chunk);
        const uint32_t lt = (uint32_t)(t - (uint64_t)c * tiles_per_chunk);
        const ps_chunk_desc d = load_desc(chunks + c);
        const uint32_t tile_base = d.reserved + lt * kTile;
        if (tile_base < d.numel) step_tile<U, true, true>(d, segs, nullptr, tile_base);
    }
}

// Staged form of the fused multi-GPU step, stage 1: the switch-side sum of one
// owned chunk's gradients is pulled into a local staging buffer.  Nothing but
// loads and stores, so a thread keeps kPullDepth 16-byte reduced loads in flight
// and the grid can stay small beside the step kernel.  Ragged ends (the last
// numel % 8 elements) are left to the step kernel's element-wise path, which
// reads them through the multicast mapping itself.
constexpr int kPullDepth = 8;
__global__ void __launch_bounds__(kThreads)
fused_pull_kernel(const ps_chunk_desc* __restrict__ chunk, const ps_step_ctrl* __restrict__ ctrl,
                  uint16_t* __restrict__ staging, long long mc_delta)
{
    if (__ldg(&ctrl->skip)) return;  // a skipped step restores from the master: no gradients needed
    const ps_chunk_desc d = load_desc(chunk);
    const uint32_t n_vec = d.numel / kVec;
    const char* src = reinterpret_cast<const char*>(d.h16) + mc_delta;
    const uint32_t stride = gridDim.x * kThreads;
    for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < n_vec; i += stride * kPullDepth) {
        uint4 q[kPullDepth];
#pragma unroll
        for (int k = 0; k < kPullDepth; ++k) {
            const uint32_t j = i + (uint32_t)k * stride;
            if (j < n_vec) q[k] = mm_ld_reduce_f16x8(src + (size_t)j * 16);
        }
#pragma unroll
        for (int k = 0; k < kPullDepth; ++k) {
            const uint32_t j = i + (uint32_t)k * stride;
            if (j < n_vec) reinterpret_cast<uint4*>(staging)[j] = q[k];
        }
    }
}

// Stage 2: the chunk step with the reduced gradients taken from the staging
// buffer and the fp16 params stored to every rank through the multicast mapping.
template <int U>
__global__ void __launch_bounds__(kThreads)
chunk_step_staged_kernel(const ps_chunk_desc* __restrict__ chunk, uint32_t tiles_per_chunk,
                         const ps_segment* __restrict__ segs, const ps_step_ctrl* __restrict__ ctrl,
                         const uint16_t* __restrict__ staging, McCtx mc)
{
    constexpr uint32_t kTile = kThreads * kVec * U;
    const int skip = __ldg(&ctrl->skip);
    const ps_hyper_slot* slots = ctrl->slots;
    const ps_chunk_desc d = load_desc(chunk);
    for (uint32_t lt = blockIdx.x; lt < tiles_per_chunk; lt += gridDim.x) {
        const uint32_t tile_base = lt * kTile;
        if (tile_base >= d.numel) continue;
        if (skip) {
            step_tile<U, true, true, 1, false>(d, segs, slots, tile_base, mc);
        } else {
            uint4 g[U];
#pragma unroll
            for (int j = 0; j < U; ++j) {
                const uint32_t e = tile_base + (uint32_t)(j * kThreads + threadIdx.x) * kVec;
                g[j] = make_uint4(0u, 0u, 0u, 0u);
                if (e + kVec <= d.numel) g[j] = ld_stream(reinterpret_cast<const uint4*>(staging + e));
            }
            step_tile<U, false, true, 1, true>(d, segs, slots, tile_base, mc, g);
        }
    }
    __threadfence_system();
}

// Parameters managed by torch (fp32 parameter = master, fp32 gradient, no fp16
// slot; fp16_cpu_adam.py:345-353): the whole table in one launch.  Tiles of
// kThreads * 4 elements are numbered tensor-major.  The gradient is unscaled and
// (when clipping is on) clamped in fp32, as the reference's clamp_ on the fp32
// grad tensor does; it is not divided by the world size.
__global__ void __launch_bounds__(kThreads)
tensor_table_step_kernel(const ps_tensor_desc* __restrict__ tensors, uint32_t n_tensors,
                         uint32_t tiles_per_tensor, const ps_step_ctrl* __restrict__ ctrl)
{
    if (__ldg(&ctrl->skip)) return;
    constexpr uint32_t kTile = kThreads * 4;
    const uint64_t total = (uint64_t)n_tensors * tiles_per_tensor;
    for (uint64_t t = blockIdx.x; t < total; t += gridDim.x) {
        const uint32_t c = (uint32_t)(t / tiles_per_tensor);
        const uint64_t lt = t - (uint64_t)c * tiles_per_tensor;
        const ps_tensor_desc d = tensors[c];
        const uint64_t e = lt * kTile + (uint64_t)threadIdx.x * 4;
        if (e >= d.numel) continue;
        const Slot s = load_slot(ctrl->slots + d.slot);
        const bool vec = ((reinterpret_cast<uintptr_t>(d.p32) | reinterpret_cast<uintptr_t>(d.grad) |
                           reinterpret_cast<uintptr_t>(d.exp_avg) |
                           reinterpret_cast<uintptr_t>(d.exp_avg_sq)) & 15u) == 0 && e + 4 <= d.numel;
        if (vec) {
            const float4 gq = ld_stream(reinterpret_cast<const float4*>(d.grad + e));
            const float4 pq = ld_stream(reinterpret_cast<const float4*>(d.p32 + e));
            const float4 mq = ld_stream(reinterpret_cast<const float4*>(d.exp_avg + e));
            const float4 vq = ld_stream(reinterpret_cast<const float4*>(d.exp_avg_sq + e));
            float g[4] = {gq.x, gq.y, gq.z, gq.w}, pp[4] = {pq.x, pq.y, pq.z, pq.w};
            float m[4] = {mq.x, mq.y, mq.z, mq.w}, v[4] = {vq.x, vq.y, vq.z, vq.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (s.clip > 0.f) g[k] = clamp_keep_nan(g[k], s.clip);
                adam_element(g[k], pp[k], m[k], v[k], s);
            }
            st_stream(reinterpret_cast<float4*>(d.p32 + e), make_float4(pp[0], pp[1], pp[2], pp[3]));
            st_stream(reinterpret_cast<float4*>(d.exp_avg + e), make_float4(m[0], m[1], m[2], m[3]));
            st_stream(reinterpret_cast<float4*>(d.exp_avg_sq + e), make_float4(v[0], v[1], v[2], v[3]));
        } else {
            const uint64_t e_end = e + 4 < d.numel ? e + 4 : d.numel;
            for (uint64_t i = e; i < e_end; ++i) {
                float g = d.grad[i], pp = d.p32[i], m = d.exp_avg[i], v = d.exp_avg_sq[i];
                if (s.clip > 0.f) g = clamp_keep_nan(g, s.clip);
                adam_element(g, pp, m, v, s);
                d.p32[i] = pp;
                d.exp_avg[i] = m;
                d.exp_avg_sq[i] = v;
            }
        }
    }
}

// dst[i] = the peer-to-peer kernel's reduced gradient of the element at byte
// offset 2*i from `local_ptr` in this rank's buffer; for tests.
__global__ void __launch_bounds__(kThreads)
p2p_reduce_probe_kernel(const uint16_t* local_ptr, uint16_t* dst, size_t n, McCtx mc)
{
    const size_t n_vec = n / kVec;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n_vec;
         i += (size_t)gridDim.x * kThreads)
        reinterpret_cast<uint4*>(dst)[i] = p2p_ld_reduce_f16x8<kMaxPeers>(local_ptr + i * kVec, mc);
    if (blockIdx.x == 0)
        for (size_t i = n_vec * kVec + threadIdx.x; i < n; i += kThreads)
            dst[i] = (uint16_t)p2p_ld_reduce_f16(local_ptr + i, mc);
}

// dst[i] = sum over ranks of their fp16 buffers at the multicast address mc[i]
// (what the fused kernel's gradient load returns); for tests.
__global__ void __launch_bounds__(kThreads)
multimem_reduce_probe_kernel(const uint16_t* mc, uint16_t* dst, size_t n)
{
    const size_t n_vec = n / kVec;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n_vec;
         i += (size_t)gridDim.x * kThreads)
        reinterpret_cast<uint4*>(dst)[i] = mm_ld_reduce_f16x8(mc + i * kVec);
    if (blockIdx.x == 0)
        for (size_t i = n_vec * kVec + threadIdx.x; i < n; i += kThreads)
        {
            McCtx ctx;
            ctx.mc_delta = 0;  // `mc` already is the multicast address
            ctx.peers = nullptr;
            ctx.gather = nullptr;
            ctx.local_base = nullptr;
            ctx.world = 0;
            dst[i] = (uint16_t)mm_ld_reduce_f16(mc + i, ctx);
        }
}

// Tensor-level variant (image of adam_update): `d` holds the four pointers
// advanced past `head` (0..7) leading elements so that all of them are 16-byte
// aligned; d.numel counts the elements from there on.  The leading elements are
// updated one per thread by block 0.
template <int U, bool kWrite16>
__global__ void __launch_bounds__(kThreads)
tensor_step_kernel(ps_chunk_desc d, uint32_t head, ps_hyper_slot slot, uint32_t n_tiles)
{
    constexpr uint32_t kTile = kThreads * kVec * U;
    __shared__ __align__(16) ps_segment s_seg;
    __shared__ __align__(16) ps_hyper_slot s_slot;
    if (threadIdx.x == 0) {
        s_seg = ps_segment{0u, d.numel, 0u, 0u};
        s_slot = slot;
    }
    __syncthreads();
    d.seg_begin = 0;
    d.seg_end = 1;
    if (blockIdx.x == 0 && threadIdx.x < head) {
        const Slot s = slot_from_value(slot);
        const int i = -(int)head + (int)threadIdx.x;
        float p = d.p32[i], m = d.exp_avg[i], v = d.exp_avg_sq[i];
        adam_element(grad_from_half(d.h16[i], s), p, m, v, s);
        d.p32[i] = p;
        d.exp_avg[i] = m;
        d.exp_avg_sq[i] = v;
        if (kWrite16) d.h16[i] = (uint16_t)float_to_half_bits(p);
    }
    for (uint32_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        const uint32_t tile_base = t * kTile;
        if (tile_base >= d.numel) continue;
        step_tile<U, false, kWrite16>(d, &s_seg, &s_slot, tile_base);
    }
}

// Element-wise kernel for adam_update arguments the vector path cannot take:
// fp32 gradients, a separate fp16 output, or pointers that are not mutually
// 16-byte co-aligned.
template <bool kGradHalf>
__global__ void __launch_bounds__(kThreads)
tensor_step_scalar_kernel(float* p32, const void* grads, float* exp_avg, float* exp_avg_sq, size_t n,
                          ps_hyper_slot slot, uint16_t* p16_out)
{
    const Slot s = slot_from_value(slot);
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n;
         i += (size_t)gridDim.x * kThreads) {
        float g;
        if (kGradHalf)
            g = grad_from_half(reinterpret_cast<const uint16_t*>(grads)[i], s);
        else
            g = reinterpret_cast<const float*>(grads)[i];
        float p = p32[i], m = exp_avg[i], v = exp_avg_sq[i];
        adam_element(g, p, m, v, s);
        p32[i] = p;
        exp_avg[i] = m;
        exp_avg_sq[i] = v;
        if (p16_out) p16_out[i] = (uint16_t)float_to_half_bits(p);
    }
}

// inf/nan test on packed halves: a half is inf or nan when its five exponent
// bits are all set.
__device__ __forceinline__ uint32_t nonfinite2(uint32_t w)
{
    return __vcmpeq2(w & 0x7c007c00u, 0x7c007c00u);
}

template <int U>
__global__ void __launch_bounds__(kThreads)
overflow_scan_kernel(const ps_chunk_desc* __restrict__ chunks, uint32_t n_chunks,
                     uint32_t tiles_per_chunk, int32_t* __restrict__ flag)
{
    constexpr uint32_t kTile = kThreads * kVec * U;
    uint32_t found = 0;
    const uint64_t total = (uint64_t)n_chunks * tiles_per_chunk;
    for (uint64_t t = blockIdx.x; t < total; t += gridDim.x) {
        const uint32_t c = (uint32_t)(t / tiles_per_chunk);
        const uint32_t lt = (uint32_t)(t - (uint64_t)c * tiles_per_chunk);
        const uint16_t* h16 = reinterpret_cast<const uint16_t*>(
            __ldg(reinterpret_cast<const unsigned long long*>(&chunks[c].h16)));
        const uint32_t numel = __ldg(&chunks[c].numel);
        const uint32_t tile_base = lt * kTile;
        if (tile_base >= numel) continue;
        uint4 q[U];
        uint32_t e[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            e[j] = tile_base + (uint32_t)(j * kThreads + threadIdx.x) * kVec;
            q[j] = make_uint4(0, 0, 0, 0);
            if (e[j] + kVec <= numel) q[j] = ld_stream(reinterpret_cast<const uint4*>(h16 + e[j]));
        }
#pragma unroll
        for (int j = 0; j < U; ++j) {
            found |= nonfinite2(q[j].x) | nonfinite2(q[j].y) | nonfinite2(q[j].z) | nonfinite2(q[j].w);
            if (e[j] < numel && e[j] + kVec > numel) {
                for (uint32_t i = e[j]; i < numel; ++i) found |= ((h16[i] & 0x7c00u) == 0x7c00u);
            }
        }
    }
    if (__syncthreads_or(found != 0) && threadIdx.x == 0) atomicOr(flag, 1);
}

template <int U>
__global__ void __launch_bounds__(kThreads)
overflow_scan_buffer_kernel(const uint16_t* __restrict__ g, size_t n, size_t head, int32_t* flag)
{
    // [0, head) and the ragged tail are read element-wise by block 0; the
    // 16-byte aligned body [head, head + 8 * n_vec) is read as uint4.
    uint32_t found = 0;
    const size_t n_vec = (n - head) / kVec;
    const uint4* body = reinterpret_cast<const uint4*>(g + head);
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n_vec;
         i += (size_t)gridDim.x * kThreads) {
        uint4 q = ld_stream(body + i);
        found |= nonfinite2(q.x) | nonfinite2(q.y) | nonfinite2(q.z) | nonfinite2(q.w);
    }
    if (blockIdx.x == 0) {
        for (size_t i = threadIdx.x; i < head; i += kThreads) found |= ((g[i] & 0x7c00u) == 0x7c00u);
        for (size_t i = head + n_vec * kVec + threadIdx.x; i < n; i += kThreads)
            found |= ((g[i] & 0x7c00u) == 0x7c00u);
    }
    if (__syncthreads_or(found != 0) && threadIdx.x == 0) atomicOr(flag, 1);
}

// Gradient hand-off of the backward pass (patrickstar/core/hook.py:212-216): the
// parameter's fp16 gradient is tested for inf/nan and copied into the
// parameter's fp16 slot in ONE pass (2 B read + 2 B written per element), so the
// step needs no separate scan of these elements.
__global__ void __launch_bounds__(kThreads)
grad_handoff_kernel(const uint16_t* __restrict__ g, uint16_t* __restrict__ slot, size_t n, size_t head,
                    int vec_ok, int32_t* flag)
{
    uint32_t found = 0;
    if (vec_ok) {
        const size_t n_vec = (n - head) / kVec;
        const uint4* src = reinterpret_cast<const uint4*>(g + head);
        uint4* dst = reinterpret_cast<uint4*>(slot + head);
        for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n_vec;
             i += (size_t)gridDim.x * kThreads) {
            uint4 q = ld_stream(src + i);
            found |= nonfinite2(q.x) | nonfinite2(q.y) | nonfinite2(q.z) | nonfinite2(q.w);
            dst[i] = q;
        }
        if (blockIdx.x == 0) {
            for (size_t i = threadIdx.x; i < head; i += kThreads) {
                uint16_t h = g[i];
                found |= ((h & 0x7c00u) == 0x7c00u);
                slot[i] = h;
            }
            for (size_t i = head + n_vec * kVec + threadIdx.x; i < n; i += kThreads) {
                uint16_t h = g[i];
                found |= ((h & 0x7c00u) == 0x7c00u);
                slot[i] = h;
            }
        }
    } else {
        for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n;
             i += (size_t)gridDim.x * kThreads) {
            uint16_t h = g[i];
            found |= ((h & 0x7c00u) == 0x7c00u);
            slot[i] = h;
        }
    }
    if (__syncthreads_or(found != 0) && threadIdx.x == 0 && flag != nullptr) atomicOr(flag, 1);
}

// ---------------------------------------------------------------------------
// step-begin: skip decision, step counter, beta^t history, hyper slots,
// loss-scale update.  One thread.
// ---------------------------------------------------------------------------
__device__ void derive_slot(ps_hyper_slot* out, const ps_group_hyper& g, float b1t, float b2t,
                            int bias_correction, float loss_scale, float clip, float divisor)
{
    // update_state (cpu_adam.h:163-175)
    float bc1 = 1.0f, bc2 = 1.0f;
    if (bias_correction == 1) {
        bc1 = __fsub_rn(1.0f, b1t);
        bc2 = __fdiv_rn(1.0f, __fsqrt_rn(__fsub_rn(1.0f, b2t)));
    }
    // Adam_Optimizer::Step prologue (cpu_adam.cpp:42-46)
    out->loss_scale = loss_scale;
    out->beta1 = g.beta1;
    out->beta2 = g.beta2;
    out->beta1_minus1 = __fsub_rn(1.0f, g.beta1);
    out->beta2_minus1 = __fsub_rn(1.0f, g.beta2);
    out->bias2_sqrt = bc2;
    out->eps = g.eps;
    out->step_size = __fdiv_rn(-g.lr, bc1);
    out->weight_decay = g.weight_decay;
    out->w_decay = __fmul_rn(-g.lr, g.weight_decay);
    out->clip = clip;
    out->grad_divisor = divisor;
    out->adamw_mode = g.adamw_mode;
    out->inv_loss_scale = loss_scale > 0.f ? exact_reciprocal_or_zero(loss_scale) : 0.f;
    out->inv_grad_divisor = divisor > 1.f ? __fdiv_rn(1.0f, divisor) : 0.f;
    out->reserved = 0;
}

__device__ void pow_lookup(const float* tab, uint64_t tab_len, int group, uint64_t t, float beta1,
                           float beta2, float* b1t, float* b2t, int32_t* error)
{
    if (tab != nullptr && t < tab_len) {
        const float* e = tab + 2 * ((uint64_t)group * tab_len + t);
        *b1t = e[0];
        *b2t = e[1];
    } else {
        // the host keeps the table ahead of the step counter; reaching this is a
        // host bug, reported through the sticky error word
        *error |= 1;
        *b1t = (float)pow((double)beta1, (double)t);
        *b2t = (float)pow((double)beta2, (double)t);
    }
}

// DynamicLossScaler.update_scale (loss_scaler.py:158-182)
__device__ void scaler_update(ps_scaler_state* sc, int overflow)
{
    if (sc->dynamic <= 0) return;
    if (overflow) {
        if (sc->delayed_shift == 1 || sc->cur_hysteresis == 1) {
            sc->cur_scale = fmax(sc->cur_scale / sc->scale_factor, sc->min_scale);
        } else {
            sc->cur_hysteresis -= 1;
        }
        sc->last_overflow_iter = sc->cur_iter;
    } else {
        if (sc->consecutive_hysteresis) sc->cur_hysteresis = sc->delayed_shift;
        if ((sc->cur_iter - sc->last_overflow_iter) % sc->scale_window == 0) {
            if (!sc->consecutive_hysteresis) sc->cur_hysteresis = sc->delayed_shift;
            sc->cur_scale *= sc->scale_factor;
        }
    }
    sc->cur_iter += 1;
}

__global__ void scaler_update_kernel(ps_scaler_state* sc, int32_t* flag, int overflow_host)
{
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int overflow = flag != nullptr ? (*flag != 0) : (overflow_host != 0);
    scaler_update(sc, overflow);
    if (flag != nullptr) *flag = 0;
}

__global__ void step_begin_kernel(ps_step_ctrl* ctrl, ps_scaler_state* sc, int32_t* flag,
                                  ps_step_plan plan, const float* pow_tab, uint64_t tab_len)
{
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    // FP16Adam.check_overflow only ever sets the flag with a dynamic scaler
    // (LossScaler.has_overflow is constant False, loss_scaler.py:61-62)
    int overflow = (sc->dynamic > 0 && flag != nullptr && *flag != 0) ? 1 : 0;
    const float loss_scale = (sc->dynamic < 0) ? -1.0f : (float)sc->cur_scale;
    float clip = 0.f;
    if (plan.clip > 0.0) {
        double c = plan.clip;
        if (sc->dynamic >= 0) c *= sc->cur_scale;
        clip = (float)fmin(65504.0, c);
    }
    if (overflow) {
        // fp16_cpu_adam.py:549-558: early return, state["step"] untouched
        ctrl->skip = 1;
        ctrl->n_skipped += 1;
    } else {
        ctrl->skip = 0;
        const uint64_t t = ++ctrl->step;  // fp16_cpu_adam.py:574
        // first adam_update call of the step: IncrementStep (cpu_adam.h:143-162)
        const ps_group_hyper g0 = plan.groups[plan.first_group];
        float b1t = ctrl->betta1_t, b2t = ctrl->betta2_t;
        if (plan.n_calls < 1) {
            // a rank without local parameters makes no adam_update call
        } else if (g0.beta1 != ctrl->betta1 || g0.beta2 != ctrl->betta2) {
            ctrl->native_step = t;
            ctrl->betta1 = g0.beta1;
            ctrl->betta2 = g0.beta2;
            pow_lookup(pow_tab, tab_len, plan.first_group, t, g0.beta1, g0.beta2, &b1t, &b2t,
                       &ctrl->error);
        } else {
            ctrl->native_step += 1;
            if (ctrl->native_step != t) {
                pow_lookup(pow_tab, tab_len, plan.first_group, t, g0.beta1, g0.beta2, &b1t, &b2t,
                           &ctrl->error);
                ctrl->native_step = t;
            } else {
                b1t = __fmul_rn(b1t, g0.beta1);
                b2t = __fmul_rn(b2t, g0.beta2);
            }
        }
        ctrl->betta1_t = b1t;
        ctrl->betta2_t = b2t;
        derive_slot(&ctrl->slots[0], g0, b1t, b2t, plan.bias_correction, loss_scale, clip,
                    plan.grad_divisor);
        if (plan.n_calls >= 2) {
            // every later call of the step finds _step == step already, or other
            // betas: both branches recompute pow(beta, step)
            for (int g = 0; g < plan.n_groups; ++g) {
                float c1, c2;
                pow_lookup(pow_tab, tab_len, g, t, plan.groups[g].beta1, plan.groups[g].beta2, &c1,
                           &c2, &ctrl->error);
                derive_slot(&ctrl->slots[1 + g], plan.groups[g], c1, c2, plan.bias_correction,
                            loss_scale, clip, plan.grad_divisor);
                if (g == plan.last_group) {
                    ctrl->betta1 = plan.groups[g].beta1;
                    ctrl->betta2 = plan.groups[g].beta2;
                    ctrl->betta1_t = c1;
                    ctrl->betta2_t = c2;
                    ctrl->native_step = t;
                }
            }
        }
    }
    scaler_update(sc, overflow);
    if (flag != nullptr) *flag = 0;
}

__global__ void ctrl_init_kernel(ps_step_ctrl* ctrl, uint64_t step, float betta1, float betta2)
{
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    ctrl->skip = 0;
    ctrl->error = 0;
    ctrl->step = step;
    ctrl->n_skipped = 0;
    // a fresh Adam_Optimizer: _step 0, betta^t 1 (cpu_adam.h:100-103); a resumed
    // one takes the pow branch on its first call because _step + 1 != step
    ctrl->native_step = 0;
    ctrl->betta1 = betta1;
    ctrl->betta2 = betta2;
    ctrl->betta1_t = 1.0f;
    ctrl->betta2_t = 1.0f;
    ps_hyper_slot z;
    memset(&z, 0, sizeof(z));
    for (int i = 0; i < PS_MAX_SLOTS; ++i) ctrl->slots[i] = z;
}

__global__ void scaler_init_kernel(ps_scaler_state* sc, ps_scaler_state init)
{
    if (threadIdx.x == 0 && blockIdx.x == 0) *sc = init;
}

__global__ void scale_loss_kernel(const float* loss, float* out, size_t n, const ps_scaler_state* sc)
{
    // Python computes loss * cur_scale with the scale as a double scalar that
    // torch converts to the tensor's dtype
    const float s = (sc->dynamic < 0) ? 1.0f : (float)sc->cur_scale;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x)
        out[i] = __fmul_rn(loss[i], s);
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------

// Host image of Adam_Optimizer's scalar state (cpu_adam.h:93-112, 143-175).
struct AdamClock {
    float alpha, betta1, betta2, eps, weight_decay;
    float betta1_t = 1.0f, betta2_t = 1.0f;
    size_t step = 0;
    float bias_correction1 = 1.0f, bias_correction2 = 1.0f;
    bool adamw_mode = true;
    std::mutex mu;  // held across increment_step / update_state / slot of one adam_update call

    void increment_step(size_t s, float beta1, float beta2)
    {
        if (beta1 != betta1 || beta2 != betta2) {
            step = s;
            betta1 = beta1;
            betta2 = beta2;
            betta1_t = (float)std::pow((double)betta1, (double)s);
            betta2_t = (float)std::pow((double)betta2, (double)s);
        } else {
            step++;
            if (step != s) {
                betta1_t = (float)std::pow((double)betta1, (double)s);
                betta2_t = (float)std::pow((double)betta2, (double)s);
                step = s;
            } else {
                betta1_t *= betta1;
                betta2_t *= betta2;
            }
        }
    }
    void update_state(float lr, float epsilon, float wd, bool bias_correction)
    {
        alpha = lr;
        eps = epsilon;
        weight_decay = wd;
        bias_correction1 = 1.0f;
        bias_correction2 = 1.0f;
        if (bias_correction) {
            bias_correction1 = 1 - betta1_t;
            bias_correction2 = 1 / sqrtf(1 - betta2_t);
        }
    }
    ps_hyper_slot slot(float loss_scale) const
    {
        ps_hyper_slot s;
        memset(&s, 0, sizeof(s));
        s.loss_scale = loss_scale;
        s.beta1 = betta1;
        s.beta2 = betta2;
        s.beta1_minus1 = 1 - betta1;
        s.beta2_minus1 = 1 - betta2;
        s.bias2_sqrt = bias_correction2;
        s.eps = eps;
        s.step_size = -1 * alpha / bias_correction1;
        s.weight_decay = weight_decay;
        s.w_decay = -1 * alpha * weight_decay;
        s.clip = 0.f;
        s.grad_divisor = 0.f;
        s.adamw_mode = adamw_mode ? 1 : 0;
        s.inv_loss_scale = loss_scale > 0.f ? exact_reciprocal_or_zero(loss_scale) : 0.f;
        return s;
    }
};

std::mutex g_opt_mu;
std::unordered_map<int, std::shared_ptr<AdamClock>> g_optimizers;

// Grid of a streaming kernel: SM count x resident CTAs per SM (occupancy
// calculator) x `waves`.  Two waves measured 0.5 % faster than one for the
// chunk step (finer tail balancing); odd multiples of the SM count that are
// not multiples of the resident CTA count lose up to 20 %.
template <typename K>
int grid_for(K kernel, uint64_t total_tiles, int* grid_out, int waves = 1)
{
    DeviceInfo di;
    int rc = device_info(&di);
    if (rc != PS_OK) return rc;
    int per_sm = g_tune.blocks_per_sm;
    if (per_sm <= 0) {
        PS_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, 0));
        if (per_sm < 1) per_sm = 1;
        per_sm *= waves;
    }
    uint64_t g = (uint64_t)di.sm_count * (uint64_t)per_sm;
    if (g > total_tiles) g = total_tiles;
    if (g < 1) g = 1;
    *grid_out = (int)g;
    return PS_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <int U>
int launch_chunk_step(const ps_chunk_desc* chunks, uint32_t n_chunks, uint32_t max_numel,
                      const ps_segment* segs, const ps_step_ctrl* ctrl, cudaStream_t st)
{
    constexpr uint32_t kTile = kThreads * kVec * U;
    uint32_t tpc = (uint32_t)(((uint64_t)max_numel + kTile - 1) / kTile);
    uint64_t total = (uint64_t)tpc * n_chunks;
    int grid = 1;
    int rc = grid_for(chunk_step_kernel<U>, total, &grid, 2);
    if (rc != PS_OK) return rc;
    chunk_step_kernel<U><<<grid, kThreads, 0, st>>>(chunks, n_chunks, tpc, segs, ctrl);
    return after_launch();
}

template <int kBulkStages>
int launch_chunk_step_bulk(const ps_chunk_desc* chunks, uint32_t n_chunks, uint32_t max_numel,
                           const ps_segment* segs, const ps_step_ctrl* ctrl, cudaStream_t st)
{
    constexpr int kSmem = kBulkStages * (int)kBulkStageBytes;
    auto kernel = chunk_step_bulk_kernel<kBulkStages>;
    PS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    uint32_t tpc = (uint32_t)(((uint64_t)max_numel + kBulkTile - 1) / kBulkTile);
    uint64_t total = (uint64_t)tpc * n_chunks;
    DeviceInfo di;
    int rc = device_info(&di);
    if (rc != PS_OK) return rc;
    int per_sm = g_tune.blocks_per_sm;
    if (per_sm <= 0) {
        PS_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, kSmem));
        if (per_sm < 1) per_sm = 1;
    }
    uint64_t g = (uint64_t)di.sm_count * (uint64_t)per_sm;
    if (g > total) g = total;
    kernel<<<(int)g, kThreads, kSmem, st>>>(chunks, n_chunks, tpc, segs, ctrl);
    return after_launch();
}

template <int kDepth, int kMinBlocks>
int launch_chunk_step_fused(const ps_chunk_desc* chunks, uint32_t n_chunks, uint32_t max_numel,
                            const ps_segment* segs, const ps_step_ctrl* ctrl, McCtx mc, cudaStream_t st)
{
    constexpr uint32_t kTile = kThreads * kVec;
    uint32_t tpc = (uint32_t)(((uint64_t)max_numel + kTile - 1) / kTile);
    uint64_t total = (uint64_t)tpc * n_chunks;
    int grid = 1;
    const int saved = g_tune.blocks_per_sm;
    g_tune.blocks_per_sm = g_tune.fused_blocks_per_sm;
    int rc = grid_for(chunk_step_fused_kernel<kDepth, kMinBlocks>, total, &grid, 1);
    g_tune.blocks_per_sm = saved;
    if (rc != PS_OK) return rc;
    chunk_step_fused_kernel<kDepth, kMinBlocks><<<grid, kThreads, 0, st>>>(chunks, n_chunks, tpc, segs, ctrl, mc);
    return after_launch();
}

template <int U, int kColl, int kMinBlocks = 2>
int launch_chunk_step_p2p(const ps_chunk_desc* chunks, uint32_t n_chunks, uint32_t max_numel,
                          const ps_segment* segs, const ps_step_ctrl* ctrl, McCtx mc, cudaStream_t st)
{
    constexpr uint32_t kTile = kThreads * kVec * U;
    uint32_t tpc = (uint32_t)(((uint64_t)max_numel + kTile - 1) / kTile);
    int grid = 1;
    const int saved = g_tune.blocks_per_sm;
    g_tune.blocks_per_sm = g_tune.p2p_blocks_per_sm;
    int rc = grid_for(chunk_step_p2p_kernel<U, kColl, kMinBlocks>, (uint64_t)tpc * n_chunks, &grid, 2);
    g_tune.blocks_per_sm = saved;
    if (rc != PS_OK) return rc;
    chunk_step_p2p_kernel<U, kColl, kMinBlocks><<<grid, kThreads, 0, st>>>(chunks, n_chunks, tpc, segs, ctrl, mc);
    return after_launch();
}

template <int U>
int launch_chunk_restore(const ps_chunk_desc* chunks, uint32_t n_chunks, uint32_t max_numel,
                         const ps_segment* segs, cudaStream_t st)
{
    constexpr uint32_t kTile = kThreads * kVec * U;
    uint32_t tpc = (uint32_t)(((uint64_t)max_numel + kTile - 1) / kTile);
    int grid = 1;
    int rc = grid_for(chunk_restore_kernel<U>, (uint64_t)tpc * n_chunks, &grid, 2);
    if (rc != PS_OK) return rc;
    chunk_restore_kernel<U><<<grid, kThreads, 0, st>>>(chunks, n_chunks, tpc, segs);
    return after_launch();
}

// Streams and events of ps_chunk_step_copy (two staging slots, one pull and one push stream
// per peer so that the copies to and from different peers run on different copy engines).
constexpr int kCopyMaxSlots = 8;
struct CopyPipe {
    int device = -1;
    int n_slots = 2;
    cudaStream_t pull[kMaxPeers] = {}, push[kMaxPeers] = {};
    cudaEvent_t start = nullptr, stepped[kCopyMaxSlots] = {};
    cudaEvent_t pulled[kCopyMaxSlots][kMaxPeers] = {}, pushed[kMaxPeers] = {};
};

// Stream and events of ps_chunk_step_fused_staged (two staging slots).
struct FusedPipe {
    int device = -1;
    cudaStream_t pull = nullptr;
    cudaEvent_t start = nullptr, full[2] = {nullptr, nullptr}, freed[2] = {nullptr, nullptr};
};

template <int U, bool kWrite16>
int launch_tensor_step(const ps_chunk_desc& d, uint32_t head, const ps_hyper_slot& slot,
                       cudaStream_t st)
{
    constexpr uint32_t kTile = kThreads * kVec * U;
    uint32_t tiles = (uint32_t)(((uint64_t)d.numel + kTile - 1) / kTile);
    int grid = 1;
    int rc = grid_for(tensor_step_kernel<U, kWrite16>, tiles ? tiles : 1, &grid);
    if (rc != PS_OK) return rc;
    tensor_step_kernel<U, kWrite16><<<grid, kThreads, 0, st>>>(d, head, slot, tiles);
    return after_launch();
}

template <bool kWrite16>
int launch_tensor_step_u(const ps_chunk_desc& d, uint32_t head, const ps_hyper_slot& slot,
                         cudaStream_t st)
{
    switch (g_tune.unroll) {
        case 1: return launch_tensor_step<1, kWrite16>(d, head, slot, st);
        case 4: return launch_tensor_step<4, kWrite16>(d, head, slot, st);
        default: return launch_tensor_step<2, kWrite16>(d, head, slot, st);
    }
}

template <int U>
int launch_scan(const ps_chunk_desc* chunks, uint32_t n_chunks, uint32_t max_numel, int32_t* flag,
                cudaStream_t st)
{
    constexpr uint32_t kTile = kThreads * kVec * U;
    uint32_t tpc = (uint32_t)(((uint64_t)max_numel + kTile - 1) / kTile);
    uint64_t total = (uint64_t)tpc * n_chunks;
    int grid = 1;
    int rc = grid_for(overflow_scan_kernel<U>, total, &grid);
    if (rc != PS_OK) return rc;
    overflow_scan_kernel<U><<<grid, kThreads, 0, st>>>(chunks, n_chunks, tpc, flag);
    return after_launch();
}

// ---------------------------------------------------------------------------
// scratch of ps_chunk_step_static: control block, chunk table and segment table
// of one call, resident in every context that loads this library.
// ---------------------------------------------------------------------------
constexpr size_t kStaticCtrlBytes = 1280;  // sizeof(ps_step_ctrl) rounded up to 256
constexpr size_t kStaticChunkBytes = (size_t)PS_STATIC_MAX_CHUNKS * sizeof(ps_chunk_desc);
constexpr size_t kStaticSegBytes = (size_t)PS_STATIC_MAX_SEGMENTS * sizeof(ps_segment);
constexpr size_t kStaticChunkOff = kStaticCtrlBytes;
constexpr size_t kStaticSegOff = kStaticChunkOff + kStaticChunkBytes;
constexpr size_t kStaticBytes = kStaticSegOff + kStaticSegBytes;
static_assert(sizeof(ps_step_ctrl) <= kStaticCtrlBytes, "control block outgrew its slot");
static_assert(kStaticChunkOff % 256 == 0 && kStaticSegOff % 256 == 0, "tables must stay aligned");

static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

// Device address of g_static_scratch on the current device.  In host code the
// symbol's name is only a handle; the address a kernel can use comes from
// cudaGetSymbolAddress, asked once per device with that device current.
int static_scratch_address(unsigned char** out)
{
    static std::mutex mu;
    static std::unordered_map<int, unsigned char*> by_device;
    int dev = 0;
    PS_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(mu);
    auto it = by_device.find(dev);
    if (it == by_device.end()) {
        unsigned char* ptr = nullptr;
        PS_CUDA(cudaGetSymbolAddress((void**)&ptr, g_static_scratch));
        if (ptr == nullptr) return PS_ERR_CUDA;
        it = by_device.emplace(dev, ptr).first;
    }
    *out = it->second;
    return PS_OK;
}

}  // namespace

// ---------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------
extern "C" {

int ps_version(void) { return 100; }

const char* ps_strerror(int code)
{
    switch (code) {
        case PS_OK: return "ok";
        case PS_ERR_INVALID: return "invalid argument";
        case PS_ERR_UNKNOWN_ID: return "unknown optimizer id";
        case PS_ERR_ALIGN: return "pointer or offset not aligned as required";
        case PS_ERR_CUDA: return "CUDA runtime call failed (see ps_last_cuda_error)";
        case PS_ERR_TABLE: return "chunk/segment table failed validation";
        case PS_ERR_LIMIT: return "stated maximum exceeded";
        default: return "unknown error code";
    }
}

int ps_last_cuda_error(void) { return g_last_cuda_error; }

uint64_t ps_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int ps_tune(const char* key, int value)
{
    if (key == nullptr) return PS_ERR_INVALID;
    if (!strcmp(key, "unroll")) {
        if (value != 1 && value != 2 && value != 4) return PS_ERR_INVALID;
        g_tune.unroll = value;
    } else if (!strcmp(key, "blocks_per_sm")) {
        if (value < 0 || value > 32) return PS_ERR_INVALID;
        g_tune.blocks_per_sm = value;
    } else if (!strcmp(key, "bulk")) {
        if (value != 0 && (value < 2 || value > 4)) return PS_ERR_INVALID;
        g_tune.bulk = value;
    } else if (!strcmp(key, "fused_depth")) {
        if (value != 2 && value != 4 && value != 8) return PS_ERR_INVALID;
        g_tune.fused_depth = value;
    } else if (!strcmp(key, "fused_blocks_per_sm")) {
        if (value < 0 || value > 32) return PS_ERR_INVALID;
        g_tune.fused_blocks_per_sm = value;
    } else if (!strcmp(key, "pull_blocks_per_sm")) {
        if (value < 0 || value > 32) return PS_ERR_INVALID;
        g_tune.pull_blocks_per_sm = value;
    } else if (!strcmp(key, "staged_blocks_per_sm")) {
        if (value < 0 || value > 32) return PS_ERR_INVALID;
        g_tune.staged_blocks_per_sm = value;
    } else if (!strcmp(key, "p2p_blocks_per_sm")) {
        if (value < 0 || value > 32) return PS_ERR_INVALID;
        g_tune.p2p_blocks_per_sm = value;
    } else if (!strcmp(key, "fused_min_blocks")) {
        if (value < 2 || value > 4) return PS_ERR_INVALID;
        g_tune.fused_min_blocks = value;
    } else if (!strcmp(key, "p2p_min_blocks")) {
        if (value < 2 || value > 4) return PS_ERR_INVALID;
        g_tune.p2p_min_blocks = value;
    } else if (!strcmp(key, "p2p_unroll")) {
        if (value != 0 && value != 1 && value != 2) return PS_ERR_INVALID;
        g_tune.p2p_unroll = value;
    } else if (!strcmp(key, "scan_unroll")) {
        if (value != 1 && value != 2 && value != 4) return PS_ERR_INVALID;
        g_tune.scan_unroll = value;
    } else {
        return PS_ERR_INVALID;
    }
    return PS_OK;
}

int ps_adam_create(int optimizer_id, float alpha, float betta1, float betta2, float eps,
                   float weight_decay, int adamw_mode, int should_log)
{
    auto c = std::make_shared<AdamClock>();
    c->alpha = alpha;
    c->betta1 = betta1;
    c->betta2 = betta2;
    c->eps = eps;
    c->weight_decay = weight_decay;
    c->adamw_mode = adamw_mode != 0;
    {
        std::lock_guard<std::mutex> lk(g_opt_mu);
        g_optimizers[optimizer_id] = c;
    }
    if (should_log) {
        printf("Adam Optimizer #%d is created with sm_100a CUDA arithmetic capability.\n",
               optimizer_id);
        printf("Config: alpha=%f, betas=(%f, %f), weight_decay=%f, adam_w=%d\n", alpha, betta1,
               betta2, weight_decay, adamw_mode ? 1 : 0);
    }
    return PS_OK;
}

int ps_adam_destroy(int optimizer_id)
{
    std::lock_guard<std::mutex> lk(g_opt_mu);
    return g_optimizers.erase(optimizer_id) ? PS_OK : PS_ERR_UNKNOWN_ID;
}

int ps_adam_get_state(int optimizer_id, float out[4], uint64_t* step)
{
    if (out == nullptr || step == nullptr) return PS_ERR_INVALID;
    std::lock_guard<std::mutex> lk(g_opt_mu);
    auto it = g_optimizers.find(optimizer_id);
    if (it == g_optimizers.end()) return PS_ERR_UNKNOWN_ID;
    std::lock_guard<std::mutex> lk2(it->second->mu);
    out[0] = it->second->betta1_t;
    out[1] = it->second->betta2_t;
    out[2] = it->second->bias_correction1;
    out[3] = it->second->bias_correction2;
    *step = it->second->step;
    return PS_OK;
}

int ps_adam_update(int optimizer_id, size_t step, float lr, float beta1, float beta2, float epsilon,
                   float weight_decay, int bias_correction, float* params_dev, const void* grads_dev,
                   float* exp_avg_dev, float* exp_avg_sq_dev, size_t n, int g_is_half,
                   float loss_scale, uint16_t* p16_out_dev, void* stream)
{
    std::shared_ptr<AdamClock> clock;
    {
        std::lock_guard<std::mutex> lk(g_opt_mu);
        auto it = g_optimizers.find(optimizer_id);
        if (it == g_optimizers.end()) return PS_ERR_UNKNOWN_ID;
        clock = it->second;
    }
    if (n > 0 && (params_dev == nullptr || grads_dev == nullptr || exp_avg_dev == nullptr ||
                  exp_avg_sq_dev == nullptr))
        return PS_ERR_INVALID;
    if (n >= 0x7fffff00ull) return PS_ERR_LIMIT;
    const uintptr_t pa = (uintptr_t)params_dev, ma = (uintptr_t)exp_avg_dev,
                    va = (uintptr_t)exp_avg_sq_dev, ga = (uintptr_t)grads_dev,
                    oa = (uintptr_t)p16_out_dev;
    if ((pa | ma | va) & 3u) return PS_ERR_ALIGN;
    if (g_is_half ? (ga & 1u) : (ga & 3u)) return PS_ERR_ALIGN;
    if (oa & 1u) return PS_ERR_ALIGN;
    // the history-dependent state advances even for an empty tensor, as in the
    // reference (ds_adam_step calls IncrementStep before looking at the size)
    ps_hyper_slot slot;
    {
        // two threads sharing one optimizer id must not interleave inside the beta^t history
        std::lock_guard<std::mutex> lk(clock->mu);
        clock->increment_step(step, beta1, beta2);
        clock->update_state(lr, epsilon, weight_decay, bias_correction == 1);
        slot = clock->slot(loss_scale);
    }
    if (n == 0) return PS_OK;
    cudaStream_t st = (cudaStream_t)stream;

    // Vector path: fp16 grads, fp16 output (if any) in the gradient's own
    // storage, and a common number of leading elements `head` (0..7) after
    // which all four arrays are 16-byte aligned.
    bool vector_ok = g_is_half && (p16_out_dev == nullptr || oa == ga);
    uint32_t head = 0;
    if (vector_ok) {
        head = (uint32_t)(((16u - (ga & 15u)) & 15u) >> 1);
        const uintptr_t fwd32 = (uintptr_t)head * 4u;
        vector_ok = (((pa + fwd32) | (ma + fwd32) | (va + fwd32)) & 15u) == 0;
    }
    if (vector_ok) {
        if (head > n) head = (uint32_t)n;
        ps_chunk_desc d;
        d.p32 = params_dev + head;
        d.exp_avg = exp_avg_dev + head;
        d.exp_avg_sq = exp_avg_sq_dev + head;
        d.h16 = reinterpret_cast<uint16_t*>(ga) + head;
        d.numel = (uint32_t)(n - head);
        d.seg_begin = 0;
        d.seg_end = 1;
        d.reserved = 0;
        return p16_out_dev != nullptr ? launch_tensor_step_u<true>(d, head, slot, st)
                                      : launch_tensor_step_u<false>(d, head, slot, st);
    }
    DeviceInfo di;
    int rc = device_info(&di);
    if (rc != PS_OK) return rc;
    uint64_t blocks = (n + kThreads - 1) / kThreads;
    uint64_t cap = (uint64_t)di.sm_count * 8u;
    int grid = (int)(blocks < cap ? blocks : cap);
    if (g_is_half)
        tensor_step_scalar_kernel<true><<<grid, kThreads, 0, st>>>(
            params_dev, grads_dev, exp_avg_dev, exp_avg_sq_dev, n, slot, p16_out_dev);
    else
        tensor_step_scalar_kernel<false><<<grid, kThreads, 0, st>>>(
            params_dev, grads_dev, exp_avg_dev, exp_avg_sq_dev, n, slot, p16_out_dev);
    return after_launch();
}

int ps_table_check(const ps_chunk_desc* chunks, uint32_t n_chunks, const ps_segment* segs,
                   uint32_t n_segs, uint32_t n_slots, uint32_t chunk_capacity)
{
    if (n_chunks > 0 && chunks == nullptr) return PS_ERR_INVALID;
    if (n_segs > 0 && segs == nullptr) return PS_ERR_INVALID;
    if (n_slots > PS_MAX_SLOTS) return PS_ERR_LIMIT;
    if (chunk_capacity >= 0x7fffff00u) return PS_ERR_LIMIT;
    for (uint32_t c = 0; c < n_chunks; ++c) {
        const ps_chunk_desc& d = chunks[c];
        if (!d.p32 || !d.exp_avg || !d.exp_avg_sq || !d.h16) return PS_ERR_INVALID;
        if (!aligned16(d.p32) || !aligned16(d.exp_avg) || !aligned16(d.exp_avg_sq) ||
            !aligned16(d.h16))
            return PS_ERR_ALIGN;
        if (d.numel > chunk_capacity) return PS_ERR_TABLE;
        // `reserved` is the first element the kernel touches: the 128-bit accesses start there
        if (d.reserved % 2048u != 0u) return PS_ERR_TABLE;
        if (d.reserved != 0u && d.reserved >= d.numel) return PS_ERR_TABLE;
        if (d.seg_begin > d.seg_end || d.seg_end > n_segs) return PS_ERR_TABLE;
        if (d.seg_begin == d.seg_end && d.numel != 0) return PS_ERR_TABLE;
        uint32_t prev_end = 0;
        for (uint32_t s = d.seg_begin; s < d.seg_end; ++s) {
            if (segs[s].start >= segs[s].end) return PS_ERR_TABLE;
            if (segs[s].start < prev_end) return PS_ERR_TABLE;
            if (segs[s].end > d.numel) return PS_ERR_TABLE;
            if (segs[s].slot >= n_slots) return PS_ERR_TABLE;
            prev_end = segs[s].end;
        }
    }
    return PS_OK;
}

int ps_piece_table_check(const ps_chunk_desc* pieces, uint32_t n_pieces, uint32_t n_segs, uint32_t chunk_capacity)
{
    if (n_pieces > 0 && pieces == nullptr) return PS_ERR_INVALID;
    if (chunk_capacity >= 0x7fffff00u) return PS_ERR_LIMIT;
    for (uint32_t i = 0; i < n_pieces; ++i) {
        const ps_chunk_desc& d = pieces[i];
        if (!d.p32 || !d.exp_avg || !d.exp_avg_sq || !d.h16) return PS_ERR_INVALID;
        if (!aligned16(d.p32) || !aligned16(d.exp_avg) || !aligned16(d.exp_avg_sq) || !aligned16(d.h16))
            return PS_ERR_ALIGN;
        if (d.numel > chunk_capacity) return PS_ERR_TABLE;
        if (d.reserved % 2048u != 0u || d.reserved >= d.numel) return PS_ERR_TABLE;
        if (d.seg_begin >= d.seg_end || d.seg_end > n_segs) return PS_ERR_TABLE;
    }
    return PS_OK;
}

int ps_pow_table_fill(float beta1, float beta2, uint64_t t0, uint64_t count, float* out_host)
{
    if (count > 0 && out_host == nullptr) return PS_ERR_INVALID;
    for (uint64_t i = 0; i < count; ++i) {
        out_host[2 * i] = (float)std::pow((double)beta1, (double)(size_t)(t0 + i));
        out_host[2 * i + 1] = (float)std::pow((double)beta2, (double)(size_t)(t0 + i));
    }
    return PS_OK;
}

int ps_ctrl_init(ps_step_ctrl* ctrl_dev, uint64_t step, float betta1, float betta2, void* stream)
{
    if (ctrl_dev == nullptr) return PS_ERR_INVALID;
    if (!aligned16(ctrl_dev)) return PS_ERR_ALIGN;
    ctrl_init_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(ctrl_dev, step, betta1, betta2);
    return after_launch();
}

int ps_scaler_init(ps_scaler_state* scaler_dev, const ps_scaler_state* init_host, void* stream)
{
    if (scaler_dev == nullptr || init_host == nullptr) return PS_ERR_INVALID;
    if (init_host->dynamic > 0 && (init_host->scale_window <= 0 || init_host->scale_factor <= 0.0))
        return PS_ERR_INVALID;
    scaler_init_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(scaler_dev, *init_host);
    return after_launch();
}

int ps_overflow_scan(const ps_chunk_desc* chunks_dev, uint32_t n_chunks, uint32_t max_numel,
                     int32_t* flag_dev, void* stream)
{
    if (flag_dev == nullptr) return PS_ERR_INVALID;
    if (n_chunks == 0 || max_numel == 0) return PS_OK;
    if (chunks_dev == nullptr) return PS_ERR_INVALID;
    cudaStream_t st = (cudaStream_t)stream;
    switch (g_tune.scan_unroll) {
        case 1: return launch_scan<1>(chunks_dev, n_chunks, max_numel, flag_dev, st);
        case 2: return launch_scan<2>(chunks_dev, n_chunks, max_numel, flag_dev, st);
        default: return launch_scan<4>(chunks_dev, n_chunks, max_numel, flag_dev, st);
    }
}

int ps_overflow_scan_buffer(const uint16_t* g_dev, size_t n, int32_t* flag_dev, void* stream)
{
    if (flag_dev == nullptr) return PS_ERR_INVALID;
    if (n == 0) return PS_OK;
    if (g_dev == nullptr) return PS_ERR_INVALID;
    if ((uintptr_t)g_dev & 1u) return PS_ERR_ALIGN;
    size_t head = ((16u - ((uintptr_t)g_dev & 15u)) & 15u) >> 1;
    if (head > n) head = n;
    DeviceInfo di;
    int rc = device_info(&di);
    if (rc != PS_OK) return rc;
    uint64_t n_vec = (n - head) / kVec;
    uint64_t blocks = (n_vec + kThreads - 1) / kThreads;
    uint64_t cap = (uint64_t)di.sm_count * 8u;
    int grid = (int)(blocks < cap ? blocks : cap);
    if (grid < 1) grid = 1;
    overflow_scan_buffer_kernel<1><<<grid, kThreads, 0, (cudaStream_t)stream>>>(g_dev, n, head,
                                                                               flag_dev);
    return after_launch();
}

int ps_grad_handoff(const uint16_t* grad_dev, uint16_t* slot_dev, size_t n, int32_t* flag_dev, void* stream)
{
    if (n == 0) return PS_OK;
    if (grad_dev == nullptr || slot_dev == nullptr) return PS_ERR_INVALID;
    if (((uintptr_t)grad_dev | (uintptr_t)slot_dev) & 1u) return PS_ERR_ALIGN;
    // vector path when source and slot reach a 16-byte boundary after the same number of elements
    const size_t hg = ((16u - ((uintptr_t)grad_dev & 15u)) & 15u) >> 1;
    const size_t hs = ((16u - ((uintptr_t)slot_dev & 15u)) & 15u) >> 1;
    const int vec_ok = (hg == hs);
    size_t head = hg < n ? hg : n;
    DeviceInfo di;
    int rc = device_info(&di);
    if (rc != PS_OK) return rc;
    uint64_t work = vec_ok ? (n - head) / kVec : n;
    uint64_t blocks = (work + kThreads - 1) / kThreads;
    uint64_t cap = (uint64_t)di.sm_count * 8u;
    int grid = (int)(blocks < cap ? blocks : cap);
    if (grid < 1) grid = 1;
    grad_handoff_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(grad_dev, slot_dev, n, head, vec_ok,
                                                                    flag_dev);
    return after_launch();
}

int ps_step_begin(ps_step_ctrl* ctrl_dev, ps_scaler_state* scaler_dev, int32_t* flag_dev,
                  const ps_step_plan* plan_host, const float* pow_table_dev, uint64_t pow_table_len,
                  void* stream)
{
    if (ctrl_dev == nullptr || scaler_dev == nullptr || plan_host == nullptr) return PS_ERR_INVALID;
    const ps_step_plan& p = *plan_host;
    if (p.n_groups < 1 || p.n_groups > PS_MAX_GROUPS) return PS_ERR_LIMIT;
    if (p.first_group < 0 || p.first_group >= p.n_groups || p.last_group < 0 ||
        p.last_group >= p.n_groups || p.n_calls < 0)
        return PS_ERR_INVALID;
    step_begin_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(ctrl_dev, scaler_dev, flag_dev, p,
                                                         pow_table_dev, pow_table_len);
    return after_launch();
}

int ps_scaler_update(ps_scaler_state* scaler_dev, int32_t* flag_dev, int overflow_host, void* stream)
{
    if (scaler_dev == nullptr) return PS_ERR_INVALID;
    scaler_update_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(scaler_dev, flag_dev, overflow_host);
    return after_launch();
}

int ps_chunk_step(const ps_chunk_desc* chunks_dev, uint32_t n_chunks, uint32_t max_numel,
                  const ps_segment* segs_dev, const ps_step_ctrl* ctrl_dev, void* stream)
{
    if (n_chunks == 0 || max_numel == 0) return PS_OK;
    if (chunks_dev == nullptr || segs_dev == nullptr || ctrl_dev == nullptr) return PS_ERR_INVALID;
    if (max_numel >= 0x7fffff00u) return PS_ERR_LIMIT;
    cudaStream_t st = (cudaStream_t)stream;
    switch (g_tune.bulk) {  // bulk-async staged variant, N stages deep
        case 2: return launch_chunk_step_bulk<2>(chunks_dev, n_chunks, max_numel, segs_dev, ctrl_dev, st);
        case 3: return launch_chunk_step_bulk<3>(chunks_dev, n_chunks, max_numel, segs_dev, ctrl_dev, st);
        case 4: return launch_chunk_step_bulk<4>(chunks_dev, n_chunks, max_numel, segs_dev, ctrl_dev, st);
        default: break;
    }
    switch (g_tune.unroll) {
        case 1: return launch_chunk_step<1>(chunks_dev, n_chunks, max_numel, segs_dev, ctrl_dev, st);
        case 4: return launch_chunk_step<4>(chunks_dev, n_chunks, max_numel, segs_dev, ctrl_dev, st);
        default: return launch_chunk_step<2>(chunks_dev, n_chunks, max_numel, segs_dev, ctrl_dev, st);
    }
}

int ps_chunk_step_fused(const ps_chunk_desc* chunks_dev, uint32_t n_chunks, uint32_t max_numel,
                        const ps_segment* segs_dev, const ps_step_ctrl* ctrl_dev,
                        const void* fp16_local_base, const void* fp16_multicast_base,
                        const uint64_t* peer_bases_dev, int world_size, void* stream)
{
    if (n_chunks == 0 || max_numel == 0) return PS_OK;
    if (chunks_dev == nullptr || segs_dev == nullptr || ctrl_dev == nullptr ||
        fp16_local_base == nullptr || fp16_multicast_base == nullptr || peer_bases_dev == nullptr)
        return PS_ERR_INVALID;
    if (world_size < 2 || world_size > 64) return PS_ERR_INVALID;
    if (((uintptr_t)fp16_local_base | (uintptr_t)fp16_multicast_base) & 15u) return PS_ERR_ALIGN;
    if (max_numel >= 0x7fffff00u) return PS_ERR_LIMIT;
    McCtx mc;
    mc.mc_delta = (long long)((intptr_t)fp16_multicast_base - (intptr_t)fp16_local_base);
    mc.peers = reinterpret_cast<const unsigned long long*>(peer_bases_dev);
    mc.gather = mc.peers;
    mc.local_base = reinterpret_cast<const char*>(fp16_local_base);
    mc.world = world_size;
    cudaStream_t st = (cudaStream_t)stream;
    // (reduced loads in flight per thread) x (resident CTAs per SM the register budget is cut for)
    switch (g_tune.fused_depth * 10 + g_tune.fused_min_blocks) {
        case 22: return launch_chunk_step_fused<2, 2>(chunks_dev, n_chunks, max_numel, segs_dev, ctrl_dev, mc, st);
        case 23: return launch_chunk_step_fused<2, 3>(chunks_dev, n_chunks, max_numel, segs_dev, ctrl_dev, mc, st);
        case 24: return launch_chunk_step_fused<2, 4>(chunks_dev, n_chunks, max_numel, segs_dev, ctrl_dev, mc, st);
        case 43: return launch_chunk_step_fused<4, 3>(chunks_dev, n_chunks, max_numel, segs_dev, ctrl_dev, mc, st);
        case 44: return launch_chunk_step_fused<4, 4>(chunks_dev, n_chunks, max_numel, segs_dev, ctrl_dev, mc, st);
        case 82: case 83: case 84:
            return launch_chunk_step_fused<8, 2>(chunks_dev, n_chunks, max_numel, segs_dev, ctrl_dev, mc, st);
        default: return launch_chunk_step_fused<4, 2>(chunks_dev, n_chunks, max_numel, segs_dev, ctrl_dev, mc, st);
    }
}

int ps_fused_pipe_create(void** pipe_out)
{
    if (pipe_out == nullptr) return PS_ERR_INVALID;
    auto* p = new FusedPipe();
    int rc = PS_OK;
    do {
        if (cudaGetDevice(&p->device) != cudaSuccess) { rc = PS_ERR_CUDA; break; }
        if (cudaStreamCreateWithFlags(&p->pull, cudaStreamNonBlocking) != cudaSuccess) { rc = PS_ERR_CUDA; break; }
        cudaEvent_t* evs[5] = {&p->start, &p->full[0], &p->full[1], &p->freed[0], &p->freed[1]};
        for (auto* e : evs)
            if (cudaEventCreateWithFlags(e, cudaEventDisableTiming) != cudaSuccess) { rc = PS_ERR_CUDA; break; }
    } while (0);
    if (rc != PS_OK) {
        g_last_cuda_error = (int)cudaGetLastError();
        ps_fused_pipe_destroy(p);
        return rc;
    }
    *pipe_out = p;
    return PS_OK;
}

int ps_fused_pipe_destroy(void* pipe)
{
    if (pipe == nullptr) return PS_ERR_INVALID;
    auto* p = static_cast<FusedPipe*>(pipe);
    cudaEvent_t evs[5] = {p->start, p->full[0], p->full[1], p->freed[0], p->freed[1]};
    for (auto e : evs)
        if (e) cudaEventDestroy(e);
    if (p->pull) cudaStreamDestroy(p->pull);
    delete p;
    return PS_OK;
}

int ps_chunk_step_fused_staged(void* pipe, const ps_chunk_desc* chunks_dev, uint32_t n_chunks,
                               uint32_t max_numel, const ps_segment* segs_dev, const ps_step_ctrl* ctrl_dev,
                               const void* fp16_local_base, const void* fp16_multicast_base,
                               const uint64_t* peer_bases_dev, int world_size, uint16_t* staging_dev,
                               void* stream)
{
    if (n_chunks == 0 || max_numel == 0) return PS_OK;
    if (pipe == nullptr || chunks_dev == nullptr || segs_dev == nullptr || ctrl_dev == nullptr ||
        fp16_local_base == nullptr || fp16_multicast_base == nullptr || peer_bases_dev == nullptr ||
        staging_dev == nullptr)
        return PS_ERR_INVALID;
    if (world_size < 2 || world_size > 64) return PS_ERR_INVALID;
    if (((uintptr_t)fp16_local_base | (uintptr_t)fp16_multicast_base | (uintptr_t)staging_dev) & 15u)
        return PS_ERR_ALIGN;
    if (max_numel >= 0x7fffff00u) return PS_ERR_LIMIT;
    auto* p = static_cast<FusedPipe*>(pipe);
    cudaStream_t st = (cudaStream_t)stream;
    McCtx mc;
    mc.mc_delta = (long long)((intptr_t)fp16_multicast_base - (intptr_t)fp16_local_base);
    mc.peers = reinterpret_cast<const unsigned long long*>(peer_bases_dev);
    mc.gather = mc.peers;
    mc.local_base = reinterpret_cast<const char*>(fp16_local_base);
    mc.world = world_size;
    DeviceInfo di;
    int rc = device_info(&di);
    if (rc != PS_OK) return rc;
    constexpr int U = 1;  // HBM is lightly loaded beside the links: leave the registers to the puller
    constexpr uint32_t kTile = kThreads * kVec * U;
    const uint32_t tpc = (uint32_t)(((uint64_t)max_numel + kTile - 1) / kTile);
    const int pull_grid = di.sm_count * (g_tune.pull_blocks_per_sm > 0 ? g_tune.pull_blocks_per_sm : 2);
    uint64_t step_grid = (uint64_t)di.sm_count * (g_tune.staged_blocks_per_sm > 0 ? g_tune.staged_blocks_per_sm : 1);
    if (step_grid > tpc) step_grid = tpc;
    // staging slot of chunk k: k % 2, each slot max_numel rounded up to a whole 16-byte group
    const size_t slot_elems = ((size_t)max_numel + kVec - 1) / kVec * kVec;
    PS_CUDA(cudaEventRecord(p->start, st));
    PS_CUDA(cudaStreamWaitEvent(p->pull, p->start, 0));
    for (uint32_t k = 0; k < n_chunks; ++k) {
        const int s = (int)(k & 1u);
        uint16_t* slot = staging_dev + (size_t)s * slot_elems;
        if (k >= 2) PS_CUDA(cudaStreamWaitEvent(p->pull, p->freed[s], 0));
        fused_pull_kernel<<<pull_grid, kThreads, 0, p->pull>>>(chunks_dev + k, ctrl_dev, slot, mc.mc_delta);
        rc = after_launch();
        if (rc != PS_OK) return rc;
        PS_CUDA(cudaEventRecord(p->full[s], p->pull));
        PS_CUDA(cudaStreamWaitEvent(st, p->full[s], 0));
        chunk_step_staged_kernel<U><<<(int)step_grid, kThreads, 0, st>>>(chunks_dev + k, tpc, segs_dev,
                                                                       ctrl_dev, slot, mc);
        rc = after_launch();
        if (rc != PS_OK) return rc;
        PS_CUDA(cudaEventRecord(p->freed[s], st));
    }
    return PS_OK;
}

int ps_copy_pipe_create(void** pipe_out, int n_slots)
{
    if (pipe_out == nullptr) return PS_ERR_INVALID;
    if (n_slots < 2 || n_slots > kCopyMaxSlots) return PS_ERR_INVALID;
    auto* p = new CopyPipe();
    p->n_slots = n_slots;
    bool ok = cudaGetDevice(&p->device) == cudaSuccess;
    auto ev = [&](cudaEvent_t* e) { ok = ok && cudaEventCreateWithFlags(e, cudaEventDisableTiming) == cudaSuccess; };
    ev(&p->start);
    for (int s = 0; s < n_slots; ++s) ev(&p->stepped[s]);
    for (int q = 0; q < kMaxPeers; ++q) {
        ok = ok && cudaStreamCreateWithFlags(&p->pull[q], cudaStreamNonBlocking) == cudaSuccess;
        ok = ok && cudaStreamCreateWithFlags(&p->push[q], cudaStreamNonBlocking) == cudaSuccess;
        for (int s = 0; s < n_slots; ++s) ev(&p->pulled[s][q]);
        ev(&p->pushed[q]);
    }
    if (!ok) {
        g_last_cuda_error = (int)cudaGetLastError();
        ps_copy_pipe_destroy(p);
        return PS_ERR_CUDA;
    }
    *pipe_out = p;
    return PS_OK;
}

int ps_copy_pipe_destroy(void* pipe)
{
    if (pipe == nullptr) return PS_ERR_INVALID;
    auto* p = static_cast<CopyPipe*>(pipe);
    auto ev = [](cudaEvent_t e) { if (e) cudaEventDestroy(e); };
    ev(p->start);
    for (int s = 0; s < kCopyMaxSlots; ++s) ev(p->stepped[s]);
    for (int q = 0; q < kMaxPeers; ++q) {
        for (int s = 0; s < kCopyMaxSlots; ++s) ev(p->pulled[s][q]);
        ev(p->pushed[q]);
        if (p->pull[q]) cudaStreamDestroy(p->pull[q]);
        if (p->push[q]) cudaStreamDestroy(p->push[q]);
    }
    delete p;
    return PS_OK;
}

int ps_chunk_step_copy(void* pipe, const ps_chunk_desc* chunks_dev, const ps_chunk_desc* chunks_host,
                       uint32_t n_chunks, uint32_t max_numel, const ps_segment* segs_dev,
                       const ps_step_ctrl* ctrl_dev, const void* fp16_local_base, const uint64_t* peer_bases_host,
                       const uint64_t* peer_bases_dev, int rank, int world_size, uint16_t* staging_dev,
                       uint64_t* gather_table_dev, void* stream)
{
    if (n_chunks == 0 || max_numel == 0) return PS_OK;
    if (pipe == nullptr || chunks_dev == nullptr || chunks_host == nullptr || segs_dev == nullptr ||
        ctrl_dev == nullptr || fp16_local_base == nullptr || peer_bases_host == nullptr ||
        staging_dev == nullptr || gather_table_dev == nullptr)
        return PS_ERR_INVALID;
    if (world_size < 2 || world_size > kMaxPeers) return PS_ERR_LIMIT;
    if (rank < 0 || rank >= world_size) return PS_ERR_INVALID;
    if (n_chunks > PS_COPY_MAX_CHUNKS) return PS_ERR_LIMIT;
    if (((uintptr_t)fp16_local_base | (uintptr_t)staging_dev) & 15u) return PS_ERR_ALIGN;
    if (max_numel >= 0x7fffff00u) return PS_ERR_LIMIT;
    if (peer_bases_host[rank] != (uint64_t)(uintptr_t)fp16_local_base) return PS_ERR_INVALID;
    auto* p = static_cast<CopyPipe*>(pipe);
    cudaStream_t st = (cudaStream_t)stream;
    const int W = world_size;
    const uint32_t S = (uint32_t)p->n_slots;
    const size_t slot_elems = ((size_t)max_numel + kVec - 1) / kVec * kVec;  // one peer's copy of one chunk
    auto staging_of = [&](int s, int peer_index) {
        return staging_dev + ((size_t)s * (W - 1) + peer_index) * slot_elems;
    };
    // Per chunk, per rank: the address at which the step kernel finds that rank's gradients
    // of the chunk, minus the chunk's byte offset in the fp16 buffer (the kernel adds the
    // offset of the element it works on): the own slot itself, or the staging copy.
    static thread_local std::unique_ptr<uint64_t[]> table;
    if (!table) table.reset(new (std::nothrow) uint64_t[(size_t)PS_COPY_MAX_CHUNKS * kMaxPeers]);
    if (!table) return PS_ERR_INVALID;
    for (uint32_t k = 0; k < n_chunks; ++k) {
        const uint64_t off = (uint64_t)((const char*)chunks_host[k].h16 - (const char*)fp16_local_base);
        if (((uintptr_t)chunks_host[k].h16 & 15u) != 0) return PS_ERR_ALIGN;
        int pi = 0;
        for (int r = 0; r < W; ++r) {
            if (r == rank)
                table[(size_t)k * W + r] = (uint64_t)(uintptr_t)fp16_local_base;
            else
                table[(size_t)k * W + r] = (uint64_t)(uintptr_t)staging_of((int)(k % S), pi++) - off;
        }
    }
    PS_CUDA(cudaMemcpyAsync(gather_table_dev, table.get(), (size_t)n_chunks * W * sizeof(uint64_t),
                            cudaMemcpyHostToDevice, st));
    PS_CUDA(cudaEventRecord(p->start, st));
    for (int q = 0; q < W - 1; ++q) {
        PS_CUDA(cudaStreamWaitEvent(p->pull[q], p->start, 0));
        PS_CUDA(cudaStreamWaitEvent(p->push[q], p->start, 0));
    }
    DeviceInfo di;
    int rc = device_info(&di);
    if (rc != PS_OK) return rc;
    constexpr int U = 2;
    constexpr uint32_t kTile = kThreads * kVec * U;
    for (uint32_t k = 0; k < n_chunks; ++k) {
        const int s = (int)(k % S);
        const ps_chunk_desc& d = chunks_host[k];
        const size_t off = (size_t)((const char*)d.h16 - (const char*)fp16_local_base);
        const size_t bytes = ((size_t)d.numel * 2 + 15) / 16 * 16;
        // 1. the copy engines pull every peer's gradients of this chunk into the slot's staging
        int pi = 0;
        for (int r = 0; r < W; ++r) {
            if (r == rank) continue;
            if (k >= S) PS_CUDA(cudaStreamWaitEvent(p->pull[pi], p->stepped[s], 0));  // slot free again
            if (bytes)
                PS_CUDA(cudaMemcpyAsync(staging_of(s, pi), (const char*)(uintptr_t)peer_bases_host[r] + off, bytes,
                                        cudaMemcpyDeviceToDevice, p->pull[pi]));
            PS_CUDA(cudaEventRecord(p->pulled[s][pi], p->pull[pi]));
            PS_CUDA(cudaStreamWaitEvent(st, p->pulled[s][pi], 0));
            ++pi;
        }
        // 2. sum in rank order, step, fp16 params into the own slot
        if (d.numel) {
            McCtx mc;
            mc.mc_delta = 0;
            mc.gather = reinterpret_cast<const unsigned long long*>(gather_table_dev + (size_t)k * W);
            mc.peers = peer_bases_dev ? reinterpret_cast<const unsigned long long*>(peer_bases_dev) : mc.gather;
            mc.local_base = reinterpret_cast<const char*>(fp16_local_base);
            mc.world = W;
            const uint32_t tpc = (uint32_t)(((uint64_t)d.numel + kTile - 1) / kTile);
            int grid = 1;
            // params: pushed by the copy engines afterwards (the kernel stores locally only), or
            // stored into every rank's buffer by the kernel itself when peer_bases_dev is given
            auto launch = [&](auto kernel, uint32_t tiles) -> int {
                int r2 = grid_for(kernel, tiles, &grid, 2);
                if (r2 != PS_OK) return r2;
                kernel<<<grid, kThreads, 0, st>>>(chunks_dev + k, 1, tiles, segs_dev, ctrl_dev, mc);
                return PS_OK;
            };
            const bool kernel_stores = peer_bases_dev != nullptr;
            if (W <= 2)
                rc = kernel_stores ? launch(chunk_step_p2p_kernel<U, 22, 2>, tpc) : launch(chunk_step_p2p_kernel<U, 32, 2>, tpc);
            else if (W <= 4)
                rc = kernel_stores ? launch(chunk_step_p2p_kernel<U, 24, 2>, tpc) : launch(chunk_step_p2p_kernel<U, 34, 2>, tpc);
            else
                rc = kernel_stores ? launch(chunk_step_p2p_kernel<1, 2, 2>, tpc * 2) : launch(chunk_step_p2p_kernel<1, 38, 2>, tpc * 2);
            if (rc != PS_OK) return rc;
            rc = after_launch();
            if (rc != PS_OK) return rc;
        }
        PS_CUDA(cudaEventRecord(p->stepped[s], st));
        // 3. the copy engines push the updated fp16 params into every peer's buffer
        pi = 0;
        for (int r = 0; r < W && peer_bases_dev == nullptr; ++r) {
            if (r == rank) continue;
            PS_CUDA(cudaStreamWaitEvent(p->push[pi], p->stepped[s], 0));
            if (bytes)
                PS_CUDA(cudaMemcpyAsync((char*)(uintptr_t)peer_bases_host[r] + off, (const char*)fp16_local_base + off,
                                        bytes, cudaMemcpyDeviceToDevice, p->push[pi]));
            ++pi;
        }
    }
    for (int q = 0; q < W - 1; ++q) {
        PS_CUDA(cudaEventRecord(p->pushed[q], p->push[q]));
        PS_CUDA(cudaStreamWaitEvent(st, p->pushed[q], 0));
    }
    return PS_OK;
}

int ps_restore_fp16(const ps_chunk_desc* chunks_dev, uint32_t n_chunks, uint32_t max_numel,
                    const ps_segment* segs_dev, void* stream)
{
    if (n_chunks == 0 || max_numel == 0) return PS_OK;
    if (chunks_dev == nullptr || segs_dev == nullptr) return PS_ERR_INVALID;
    if (max_numel >= 0x7fffff00u) return PS_ERR_LIMIT;
    return launch_chunk_restore<2>(chunks_dev, n_chunks, max_numel, segs_dev, (cudaStream_t)stream);
}

int ps_tensor_table_step(const ps_tensor_desc* tensors_host, uint32_t n_tensors, uint32_t n_slots,
                         ps_tensor_desc* table_dev, const ps_step_ctrl* ctrl_dev, void* stream)
{
    if (n_tensors == 0) return PS_OK;
    if (tensors_host == nullptr || table_dev == nullptr || ctrl_dev == nullptr) return PS_ERR_INVALID;
    if (n_slots > PS_MAX_SLOTS) return PS_ERR_LIMIT;
    if (n_tensors > PS_TENSOR_TABLE_MAX) return PS_ERR_LIMIT;
    if (!aligned16(table_dev)) return PS_ERR_ALIGN;
    uint64_t max_numel = 0;
    for (uint32_t i = 0; i < n_tensors; ++i) {
        const ps_tensor_desc& d = tensors_host[i];
        if (d.numel == 0) continue;
        if (!d.p32 || !d.grad || !d.exp_avg || !d.exp_avg_sq) return PS_ERR_INVALID;
        if (((uintptr_t)d.p32 | (uintptr_t)d.grad | (uintptr_t)d.exp_avg | (uintptr_t)d.exp_avg_sq) & 3u)
            return PS_ERR_ALIGN;
        if (d.slot >= n_slots) return PS_ERR_TABLE;
        if (d.numel >= (1ull << 40)) return PS_ERR_LIMIT;
        if (d.numel > max_numel) max_numel = d.numel;
    }
    if (max_numel == 0) return PS_OK;
    cudaStream_t st = (cudaStream_t)stream;
    // The gradient pointers change from step to step (autograd allocates a new .grad), so the
    // table travels with every call: through a pageable image owned by the library (one per
    // calling thread), from which cudaMemcpyAsync has taken its bytes when it returns.
    static thread_local std::unique_ptr<ps_tensor_desc[]> image;
    if (!image) image.reset(new (std::nothrow) ps_tensor_desc[PS_TENSOR_TABLE_MAX]);
    if (!image) return PS_ERR_INVALID;
    memcpy(image.get(), tensors_host, (size_t)n_tensors * sizeof(ps_tensor_desc));
    PS_CUDA(cudaMemcpyAsync(table_dev, image.get(), (size_t)n_tensors * sizeof(ps_tensor_desc),
                            cudaMemcpyHostToDevice, st));
    constexpr uint64_t kTile = kThreads * 4;
    const uint64_t tpt = (max_numel + kTile - 1) / kTile;
    if (tpt >= 0x7fffffffull) return PS_ERR_LIMIT;
    int grid = 1;
    int rc = grid_for(tensor_table_step_kernel, tpt * n_tensors, &grid, 2);
    if (rc != PS_OK) return rc;
    tensor_table_step_kernel<<<grid, kThreads, 0, st>>>(table_dev, n_tensors, (uint32_t)tpt, ctrl_dev);
    return after_launch();
}

int ps_chunk_step_p2p(const ps_chunk_desc* chunks_dev, uint32_t n_chunks, uint32_t max_numel,
                      const ps_segment* segs_dev, const ps_step_ctrl* ctrl_dev, const void* fp16_local_base,
                      const uint64_t* peer_bases_dev, int world_size, void* stream)
{
    if (n_chunks == 0 || max_numel == 0) return PS_OK;
    if (chunks_dev == nullptr || segs_dev == nullptr || ctrl_dev == nullptr || fp16_local_base == nullptr ||
        peer_bases_dev == nullptr)
        return PS_ERR_INVALID;
    if (world_size < 2 || world_size > kMaxPeers) return PS_ERR_LIMIT;
    if ((uintptr_t)fp16_local_base & 15u) return PS_ERR_ALIGN;
    if (max_numel >= 0x7fffff00u) return PS_ERR_LIMIT;
    McCtx mc;
    mc.mc_delta = 0;
    mc.peers = reinterpret_cast<const unsigned long long*>(peer_bases_dev);
    mc.gather = mc.peers;
    mc.local_base = reinterpret_cast<const char*>(fp16_local_base);
    mc.world = world_size;
    cudaStream_t st = (cudaStream_t)stream;
    // few ranks: few peer loads per group, so two groups per thread keep the link busy
    int rc;
    if (world_size <= 2 && g_tune.p2p_unroll == 2)
        rc = launch_chunk_step_p2p<2, 22>(chunks_dev, n_chunks, max_numel, segs_dev, ctrl_dev, mc, st);
    else if (world_size <= 2 && g_tune.p2p_min_blocks == 3)
        rc = launch_chunk_step_p2p<1, 22, 3>(chunks_dev, n_chunks, max_numel, segs_dev, ctrl_dev, mc, st);
    else if (world_size <= 2 && g_tune.p2p_min_blocks == 4)
        rc = launch_chunk_step_p2p<1, 22, 4>(chunks_dev, n_chunks, max_numel, segs_dev, ctrl_dev, mc, st);
    else if (world_size <= 2)   // one group per thread measured 10 % faster than two at 2 ranks
        rc = launch_chunk_step_p2p<1, 22>(chunks_dev, n_chunks, max_numel, segs_dev, ctrl_dev, mc, st);
    else if (world_size <= 4 && g_tune.p2p_min_blocks == 3)
        rc = launch_chunk_step_p2p<1, 24, 3>(chunks_dev, n_chunks, max_numel, segs_dev, ctrl_dev, mc, st);
    else if (world_size <= 4)
        rc = launch_chunk_step_p2p<1, 24>(chunks_dev, n_chunks, max_numel, segs_dev, ctrl_dev, mc, st);
    else
        rc = launch_chunk_step_p2p<1, 2>(chunks_dev, n_chunks, max_numel, segs_dev, ctrl_dev, mc, st);
    return rc;
}

int ps_p2p_reduce_probe(const void* fp16_local_ptr, const void* fp16_local_base, const uint64_t* peer_bases_dev,
                        int world_size, uint16_t* dst_dev, size_t n, void* stream)
{
    if (n == 0) return PS_OK;
    if (fp16_local_ptr == nullptr || fp16_local_base == nullptr || peer_bases_dev == nullptr || dst_dev == nullptr)
        return PS_ERR_INVALID;
    if (world_size < 2 || world_size > kMaxPeers) return PS_ERR_LIMIT;
    if (((uintptr_t)fp16_local_ptr | (uintptr_t)fp16_local_base | (uintptr_t)dst_dev) & 15u) return PS_ERR_ALIGN;
    McCtx mc;
    mc.mc_delta = 0;
    mc.peers = reinterpret_cast<const unsigned long long*>(peer_bases_dev);
    mc.gather = mc.peers;
    mc.local_base = reinterpret_cast<const char*>(fp16_local_base);
    mc.world = world_size;
    DeviceInfo di;
    int rc = device_info(&di);
    if (rc != PS_OK) return rc;
    uint64_t blocks = (n / kVec + kThreads - 1) / kThreads;
    uint64_t cap = (uint64_t)di.sm_count * 8u;
    int grid = (int)(blocks < cap ? blocks : cap);
    if (grid < 1) grid = 1;
    p2p_reduce_probe_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const uint16_t*>(fp16_local_ptr), dst_dev, n, mc);
    return after_launch();
}

int ps_multimem_reduce_probe(const void* fp16_multicast_ptr, uint16_t* dst_dev, size_t n, void* stream)
{
    if (n == 0) return PS_OK;
    if (fp16_multicast_ptr == nullptr || dst_dev == nullptr) return PS_ERR_INVALID;
    if (((uintptr_t)fp16_multicast_ptr | (uintptr_t)dst_dev) & 15u) return PS_ERR_ALIGN;
    if (n & 1u) return PS_ERR_INVALID;  // the reduced loads work on fp16 pairs
    DeviceInfo di;
    int rc = device_info(&di);
    if (rc != PS_OK) return rc;
    uint64_t blocks = (n / kVec + kThreads - 1) / kThreads;
    uint64_t cap = (uint64_t)di.sm_count * 8u;
    int grid = (int)(blocks < cap ? blocks : cap);
    if (grid < 1) grid = 1;
    multimem_reduce_probe_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const uint16_t*>(fp16_multicast_ptr), dst_dev, n);
    return after_launch();
}

int ps_scaler_read(const ps_scaler_state* scaler_dev, ps_scaler_state* out_host, void* stream)
{
    if (scaler_dev == nullptr || out_host == nullptr) return PS_ERR_INVALID;
    PS_CUDA(cudaMemcpyAsync(out_host, scaler_dev, sizeof(ps_scaler_state), cudaMemcpyDeviceToHost,
                            (cudaStream_t)stream));
    PS_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return PS_OK;
}

int ps_ctrl_read(const ps_step_ctrl* ctrl_dev, ps_step_ctrl* out_host, void* stream)
{
    if (ctrl_dev == nullptr || out_host == nullptr) return PS_ERR_INVALID;
    PS_CUDA(cudaMemcpyAsync(out_host, ctrl_dev, sizeof(ps_step_ctrl), cudaMemcpyDeviceToHost,
                            (cudaStream_t)stream));
    PS_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return PS_OK;
}

int ps_scale_loss(const float* loss_dev, float* out_dev, size_t n, const ps_scaler_state* scaler_dev,
                  void* stream)
{
    if (n == 0) return PS_OK;
    if (loss_dev == nullptr || out_dev == nullptr || scaler_dev == nullptr) return PS_ERR_INVALID;
    uint64_t blocks = (n + 255) / 256;
    int grid = (int)(blocks < 1024 ? blocks : 1024);
    scale_loss_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(loss_dev, out_dev, n, scaler_dev);
    return after_launch();
}

int ps_chunk_step_static(const ps_chunk_desc* chunks_host, uint32_t n_chunks, uint32_t max_numel,
                         const ps_segment* segs_host, uint32_t n_segs,
                         const ps_hyper_slot* slots_host, uint32_t n_slots, int skip, void* stream)
{
    if (n_chunks == 0 || max_numel == 0) return PS_OK;
    if (chunks_host == nullptr || segs_host == nullptr || slots_host == nullptr) return PS_ERR_INVALID;
    if (n_chunks > PS_STATIC_MAX_CHUNKS || n_segs > PS_STATIC_MAX_SEGMENTS || n_slots > PS_MAX_SLOTS)
        return PS_ERR_LIMIT;
    if (n_segs == 0 || n_slots == 0) return PS_ERR_INVALID;
    if (max_numel >= 0x7fffff00u) return PS_ERR_LIMIT;
    int rc = ps_table_check(chunks_host, n_chunks, segs_host, n_segs, n_slots, max_numel);
    if (rc != PS_OK) return rc;
    for (uint32_t c = 0; c < n_chunks; ++c)
        if (chunks_host[c].reserved != 0u) return PS_ERR_TABLE;  // whole chunks only here
    unsigned char* base = nullptr;
    rc = static_scratch_address(&base);  // first call on a device: cudaGetSymbolAddress
    if (rc != PS_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    // Host image of the device array, owned by the library, one per calling thread, in
    // pageable memory: a cudaMemcpyAsync from pageable memory has taken its bytes by the
    // time it returns, so neither this image nor the caller's tables (which may be pinned,
    // where the copy would be truly asynchronous) are read after this call returns.
    static thread_local std::unique_ptr<unsigned char[]> image;
    if (!image) image.reset(new (std::nothrow) unsigned char[kStaticBytes]);
    if (!image) return PS_ERR_INVALID;
    // the whole control block is rebuilt and overwritten, so nothing of the previous call
    // survives in it
    ps_step_ctrl* ctrl = reinterpret_cast<ps_step_ctrl*>(image.get());
    memset(ctrl, 0, kStaticCtrlBytes);
    ctrl->skip = skip ? 1 : 0;
    for (uint32_t i = 0; i < n_slots; ++i) ctrl->slots[i] = slots_host[i];
    const size_t chunk_bytes = (size_t)n_chunks * sizeof(ps_chunk_desc);
    const size_t seg_bytes = (size_t)n_segs * sizeof(ps_segment);
    memcpy(image.get() + kStaticChunkOff, chunks_host, chunk_bytes);
    memcpy(image.get() + kStaticSegOff, segs_host, seg_bytes);
    PS_CUDA(cudaMemcpyAsync(base, image.get(), kStaticChunkOff + chunk_bytes, cudaMemcpyHostToDevice, st));
    PS_CUDA(cudaMemcpyAsync(base + kStaticSegOff, image.get() + kStaticSegOff, seg_bytes,
                            cudaMemcpyHostToDevice, st));
    const ps_chunk_desc* chunks_dev = reinterpret_cast<const ps_chunk_desc*>(base + kStaticChunkOff);
    const ps_segment* segs_dev = reinterpret_cast<const ps_segment*>(base + kStaticSegOff);
    const ps_step_ctrl* ctrl_dev = reinterpret_cast<const ps_step_ctrl*>(base);
    switch (g_tune.unroll) {
        case 1: return launch_chunk_step<1>(chunks_dev, n_chunks, max_numel, segs_dev, ctrl_dev, st);
        case 4: return launch_chunk_step<4>(chunks_dev, n_chunks, max_numel, segs_dev, ctrl_dev, st);
        default: return launch_chunk_step<2>(chunks_dev, n_chunks, max_numel, segs_dev, ctrl_dev, st);
    }
}

}  // extern "C"
