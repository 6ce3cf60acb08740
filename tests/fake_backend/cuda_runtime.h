// Test-only stand-in for the CUDA runtime: "device" memory is host memory.  Lets the host logic of csrc/multi.cpp be
// compiled with g++ and exercised on a machine without a GPU (tests/test_multi_host_logic.py).
#pragma once
#include <cstdlib>
#include <cstring>

typedef int cudaError_t;
enum { cudaSuccess = 0, cudaErrorMemoryAllocation = 2 };
enum cudaMemcpyKind { cudaMemcpyHostToDevice = 1, cudaMemcpyDeviceToHost = 2 };

template <typename T>
inline cudaError_t cudaMalloc(T **p, size_t bytes) { *p = static_cast<T *>(std::malloc(bytes ? bytes : 1)); return *p ? cudaSuccess : cudaErrorMemoryAllocation; }
inline cudaError_t cudaFree(void *p) { std::free(p); return cudaSuccess; }
inline cudaError_t cudaMemcpy(void *dst, const void *src, size_t bytes, cudaMemcpyKind) { std::memcpy(dst, src, bytes); return cudaSuccess; }
inline cudaError_t cudaSetDevice(int) { return cudaSuccess; }
inline cudaError_t cudaGetLastError() { return cudaSuccess; }
inline const char *cudaGetErrorString(cudaError_t) { return "fake CUDA error"; }
