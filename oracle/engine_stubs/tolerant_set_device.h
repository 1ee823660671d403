// Test infrastructure, not product code.
//
// Force-included into the reference's src/engine/gpu/workspace.cc only: its constructor selects
// devices 0..3 whatever the machine has (`auto num_gpus = 4`, workspace.cc:8), which throws on a box
// with fewer GPUs.  Ordinals the machine does not have are skipped instead; nothing else changes.
#pragma once
#include <cuda_runtime.h>
static inline cudaError_t es_tolerant_set_device(int device)
{
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) return e;
    if (device >= n) return cudaSuccess;
    return cudaSetDevice(device);
}
#define cudaSetDevice es_tolerant_set_device
