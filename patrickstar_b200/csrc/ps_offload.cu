// Offload tier of the chunk optimizer step: local chunks whose fp32 master /
// momentum / variance live in pinned host memory ("hybrid" placement,
// patrickstar/ops/fp16_cpu_adam.py:523-528) are streamed through staging slots
// in HBM around the fused chunk-step kernel.
//
// The reference moves such chunks with synchronous whole-chunk copies and then
// runs its CPU Adam on them (patrickstar/ops/chunk_io_buff.py:116-126, 241-247;
// patrickstar/core/chunk_data.py:275-366).  Here the host->device copies, the
// kernel and the device->host copies of consecutive chunks overlap: three side
// streams and one event per staging slot and stage.
//
//   h2d stream : wait slot free -> copy p, m, v of chunk i into slot s -> record loaded[s]
//   kern stream: wait loaded[s] -> chunk_step over the slot            -> record updated[s]
//   d2h stream : wait updated[s] -> copy p, m, v back to the host      -> record free[s]
//
// The fp16 slot of the chunk (gradients in, fp16 params out) always stays in HBM.
// When the step is skipped on the device (overflow) the kernel only restores the
// fp16 params; the state then travels back unchanged, which costs PCIe time on a
// rare path but keeps the host free of any synchronisation.
#include "ps_b200.h"

#include <cuda_runtime.h>

#include <new>
#include <vector>

namespace {

struct Pipeline {
    int n_slots = 0;
    int device = 0;
    cudaStream_t h2d = nullptr, kern = nullptr, d2h = nullptr;
    std::vector<cudaEvent_t> loaded, updated, free_;
    cudaEvent_t begin = nullptr;
    bool primed = false;  // free_[s] has been recorded at least once
};

thread_local int g_offload_cuda_error = 0;

#define OFF_CUDA(call)                         \
    do {                                       \
        cudaError_t e__ = (call);              \
        if (e__ != cudaSuccess) {              \
            g_offload_cuda_error = (int)e__;   \
            cudaGetLastError();                \
            return PS_ERR_CUDA;                \
        }                                      \
    } while (0)

}  // namespace

extern "C" {

int ps_offload_last_cuda_error(void) { return g_offload_cuda_error; }

int ps_offload_create(void** pipeline_out, int n_slots)
{
    if (pipeline_out == nullptr) return PS_ERR_INVALID;
    if (n_slots < 1 || n_slots > PS_OFFLOAD_MAX_SLOTS) return PS_ERR_LIMIT;
    Pipeline* p = new (std::nothrow) Pipeline();
    if (p == nullptr) return PS_ERR_INVALID;
    p->n_slots = n_slots;
    cudaError_t e = cudaGetDevice(&p->device);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&p->h2d, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&p->kern, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&p->d2h, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&p->begin, cudaEventDisableTiming);
    for (int s = 0; s < n_slots && e == cudaSuccess; ++s) {
        cudaEvent_t a = nullptr, b = nullptr, c = nullptr;
        e = cudaEventCreateWithFlags(&a, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&b, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c, cudaEventDisableTiming);
        p->loaded.push_back(a);
        p->updated.push_back(b);
        p->free_.push_back(c);
    }
    if (e != cudaSuccess) {
        g_offload_cuda_error = (int)e;
        cudaGetLastError();
        ps_offload_destroy(p);
        return PS_ERR_CUDA;
    }
    *pipeline_out = p;
    return PS_OK;
}

int ps_offload_destroy(void* pipeline)
{
    Pipeline* p = static_cast<Pipeline*>(pipeline);
    if (p == nullptr) return PS_ERR_INVALID;
    for (cudaEvent_t e : p->loaded) if (e) cudaEventDestroy(e);
    for (cudaEvent_t e : p->updated) if (e) cudaEventDestroy(e);
    for (cudaEvent_t e : p->free_) if (e) cudaEventDestroy(e);
    if (p->begin) cudaEventDestroy(p->begin);
    if (p->h2d) cudaStreamDestroy(p->h2d);
    if (p->kern) cudaStreamDestroy(p->kern);
    if (p->d2h) cudaStreamDestroy(p->d2h);
    delete p;
    return PS_OK;
}

int ps_offload_step(void* pipeline, const ps_offload_chunk* chunks_host, uint32_t n_chunks,
                    float* const* staging_dev, const ps_chunk_desc* chunks_dev,
                    const ps_segment* segs_dev, const ps_step_ctrl* ctrl_dev, void* stream)
{
    Pipeline* p = static_cast<Pipeline*>(pipeline);
    if (p == nullptr) return PS_ERR_INVALID;
    if (n_chunks == 0) return PS_OK;
    if (chunks_host == nullptr || staging_dev == nullptr || chunks_dev == nullptr ||
        segs_dev == nullptr || ctrl_dev == nullptr)
        return PS_ERR_INVALID;
    for (int s = 0; s < 3 * p->n_slots; ++s)
        if (staging_dev[s] == nullptr) return PS_ERR_INVALID;
    for (uint32_t i = 0; i < n_chunks; ++i) {
        const ps_offload_chunk& c = chunks_host[i];
        if (c.p32_host == nullptr || c.exp_avg_host == nullptr || c.exp_avg_sq_host == nullptr)
            return PS_ERR_INVALID;
    }
    cudaStream_t main_stream = (cudaStream_t)stream;
    // the kernels must see the control block this step's ps_step_begin wrote
    OFF_CUDA(cudaEventRecord(p->begin, main_stream));
    OFF_CUDA(cudaStreamWaitEvent(p->kern, p->begin, 0));
    for (uint32_t i = 0; i < n_chunks; ++i) {
        const ps_offload_chunk& c = chunks_host[i];
        const int s = (int)(i % (uint32_t)p->n_slots);
        const size_t bytes = (size_t)c.numel * sizeof(float);
        float* sp = staging_dev[3 * s], *sm = staging_dev[3 * s + 1], *sv = staging_dev[3 * s + 2];
        if (p->primed || i >= (uint32_t)p->n_slots)
            OFF_CUDA(cudaStreamWaitEvent(p->h2d, p->free_[s], 0));
        if (bytes) {
            OFF_CUDA(cudaMemcpyAsync(sp, c.p32_host, bytes, cudaMemcpyHostToDevice, p->h2d));
            OFF_CUDA(cudaMemcpyAsync(sm, c.exp_avg_host, bytes, cudaMemcpyHostToDevice, p->h2d));
            OFF_CUDA(cudaMemcpyAsync(sv, c.exp_avg_sq_host, bytes, cudaMemcpyHostToDevice, p->h2d));
        }
        OFF_CUDA(cudaEventRecord(p->loaded[s], p->h2d));
        OFF_CUDA(cudaStreamWaitEvent(p->kern, p->loaded[s], 0));
        if (c.numel) {
            int rc = ps_chunk_step(chunks_dev + c.desc_index, 1, c.numel, segs_dev, ctrl_dev, p->kern);
            if (rc != PS_OK) return rc;
        }
        OFF_CUDA(cudaEventRecord(p->updated[s], p->kern));
        OFF_CUDA(cudaStreamWaitEvent(p->d2h, p->updated[s], 0));
        if (bytes) {
            OFF_CUDA(cudaMemcpyAsync(c.p32_host, sp, bytes, cudaMemcpyDeviceToHost, p->d2h));
            OFF_CUDA(cudaMemcpyAsync(c.exp_avg_host, sm, bytes, cudaMemcpyDeviceToHost, p->d2h));
            OFF_CUDA(cudaMemcpyAsync(c.exp_avg_sq_host, sv, bytes, cudaMemcpyDeviceToHost, p->d2h));
        }
        OFF_CUDA(cudaEventRecord(p->free_[s], p->d2h));
    }
    p->primed = true;
    // whoever continues on the caller's stream sees every chunk written back
    const uint32_t tail = n_chunks < (uint32_t)p->n_slots ? n_chunks : (uint32_t)p->n_slots;
    for (uint32_t s = 0; s < tail; ++s) OFF_CUDA(cudaStreamWaitEvent(main_stream, p->free_[s], 0));
    return PS_OK;
}

}  // extern "C"
