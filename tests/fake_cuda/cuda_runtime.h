// TEST INFRASTRUCTURE: a host-only stand-in for the CUDA runtime, so the engine's host logic
// (pool, buffer table, views, shape checks, error paths, trace state machine) can be compiled
// with g++ and exercised on a machine without a GPU.  "Device memory" is host memory, copies
// are memcpy, kernels are not run (the launch_* stubs in fake_kernels.cpp do nothing), streams
// and events are tokens.  Nothing here ships in libb200tt.so.
#pragma once
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef int cudaError_t;
enum { cudaSuccess = 0, cudaErrorInvalidValue = 1, cudaErrorMemoryAllocation = 2, cudaErrorNotSupported = 801 };
typedef struct fake_stream* cudaStream_t;
typedef struct fake_event* cudaEvent_t;
typedef struct fake_graph* cudaGraph_t;
typedef struct fake_exec* cudaGraphExec_t;
enum cudaMemcpyKind { cudaMemcpyHostToDevice = 1, cudaMemcpyDeviceToHost = 2, cudaMemcpyDeviceToDevice = 3 };
enum { cudaStreamNonBlocking = 1, cudaEventDisableTiming = 2 };
enum cudaStreamCaptureMode { cudaStreamCaptureModeRelaxed = 2 };
enum cudaMemoryType { cudaMemoryTypeUnregistered = 0, cudaMemoryTypeHost = 1, cudaMemoryTypeDevice = 2 };
struct cudaDeviceProp { char name[256]; int major, minor; };
struct cudaPointerAttributes { cudaMemoryType type; };

extern "C" {
// knobs the tests turn
extern uint64_t fake_cuda_memory_limit;   // bytes cudaMalloc may hand out in total (0 = unlimited)
extern uint64_t fake_cuda_memory_in_use;
extern int fake_cuda_device_count;
extern int fake_cuda_capturing;
extern int fake_cuda_current_device;
extern int fake_sync_in_capture;       // stream synchronisations asked for while a capture was open
extern int fake_smem_attr_calls[8];       // cudaFuncSetAttribute calls, by the device that was current
}
enum cudaFuncAttribute { cudaFuncAttributeMaxDynamicSharedMemorySize = 8 };

static inline const char* cudaGetErrorString(cudaError_t e) {
  return e == cudaSuccess ? "no error" : (e == cudaErrorMemoryAllocation ? "out of memory" : "fake CUDA error");
}
static inline cudaError_t cudaGetLastError() { return cudaSuccess; }
static inline cudaError_t cudaSetDevice(int d) { fake_cuda_current_device = d; return cudaSuccess; }
static inline cudaError_t cudaGetDevice(int* d) { *d = fake_cuda_current_device; return cudaSuccess; }
static inline cudaError_t cudaFuncSetAttribute(const void*, cudaFuncAttribute, int) {
  if (fake_cuda_current_device >= 0 && fake_cuda_current_device < 8) ++fake_smem_attr_calls[fake_cuda_current_device];
  return cudaSuccess;
}
static inline cudaError_t cudaGetDeviceCount(int* n) { *n = fake_cuda_device_count; return cudaSuccess; }
static inline cudaError_t cudaGetDeviceProperties(cudaDeviceProp* p, int) {
  strcpy(p->name, "fake B200"); p->major = 10; p->minor = 0; return cudaSuccess;
}
static inline cudaError_t cudaMalloc(void** p, size_t n) {
  if (fake_cuda_memory_limit && fake_cuda_memory_in_use + n > fake_cuda_memory_limit) { *p = nullptr; return cudaErrorMemoryAllocation; }
  uint64_t* raw = (uint64_t*)aligned_alloc(256, ((n + 255) / 256) * 256 + 256);
  if (!raw) return cudaErrorMemoryAllocation;
  raw[0] = n;
  fake_cuda_memory_in_use += n;
  *p = (char*)raw + 256;
  return cudaSuccess;
}
static inline cudaError_t cudaFree(void* p) {
  if (!p) return cudaSuccess;
  uint64_t* raw = (uint64_t*)((char*)p - 256);
  fake_cuda_memory_in_use -= raw[0];
  free(raw);
  return cudaSuccess;
}
static inline cudaError_t cudaMallocHost(void** p, size_t n) { *p = malloc(n ? n : 1); return *p ? cudaSuccess : cudaErrorMemoryAllocation; }
template <class T> static inline cudaError_t cudaMallocHost(T** p, size_t n) { return cudaMallocHost((void**)p, n); }
template <class T> static inline cudaError_t cudaMalloc(T** p, size_t n) { return cudaMalloc((void**)p, n); }
static inline cudaError_t cudaFreeHost(void* p) { free(p); return cudaSuccess; }
static inline cudaError_t cudaMemGetInfo(size_t* fr, size_t* tot) {
  *tot = fake_cuda_memory_limit ? fake_cuda_memory_limit : (size_t)1 << 40;
  *fr = *tot - fake_cuda_memory_in_use;
  return cudaSuccess;
}
// A captured copy does not run (as on a real stream being captured).
static inline cudaError_t cudaMemcpyAsync(void* d, const void* s, size_t n, cudaMemcpyKind, cudaStream_t) {
  if (!fake_cuda_capturing) memcpy(d, s, n);
  return cudaSuccess;
}
static inline cudaError_t cudaMemsetAsync(void* d, int v, size_t n, cudaStream_t) {
  if (!fake_cuda_capturing) memset(d, v, n);
  return cudaSuccess;
}
static inline cudaError_t cudaStreamCreateWithFlags(cudaStream_t* s, unsigned) { *s = (cudaStream_t)malloc(8); return cudaSuccess; }
static inline cudaError_t cudaStreamDestroy(cudaStream_t s) { free(s); return cudaSuccess; }
static inline cudaError_t cudaStreamSynchronize(cudaStream_t) {
  if (fake_cuda_capturing) { ++fake_sync_in_capture; return cudaErrorInvalidValue; }   // on a real stream this ends the capture in error
  return cudaSuccess;
}
static inline cudaError_t cudaEventCreate(cudaEvent_t* e) { *e = (cudaEvent_t)malloc(8); return cudaSuccess; }
static inline cudaError_t cudaEventDestroy(cudaEvent_t e) { free(e); return cudaSuccess; }
static inline cudaError_t cudaEventRecord(cudaEvent_t, cudaStream_t) { return cudaSuccess; }
static inline cudaError_t cudaEventCreateWithFlags(cudaEvent_t* e, unsigned) { *e = (cudaEvent_t)malloc(8); return cudaSuccess; }
static inline cudaError_t cudaStreamWaitEvent(cudaStream_t, cudaEvent_t, unsigned) { return cudaSuccess; }
// IPC: the fake process is alone; a handle is the pointer itself
struct cudaIpcMemHandle_t { char reserved[64]; };
enum { cudaIpcMemLazyEnablePeerAccess = 1 };
static inline cudaError_t cudaIpcGetMemHandle(cudaIpcMemHandle_t* h, void* p) { memset(h, 0, 64); memcpy(h, &p, sizeof p); return cudaSuccess; }
static inline cudaError_t cudaIpcOpenMemHandle(void** p, cudaIpcMemHandle_t h, unsigned) { memcpy(p, &h, sizeof *p); return cudaSuccess; }
static inline cudaError_t cudaIpcCloseMemHandle(void*) { return cudaSuccess; }
static inline cudaError_t cudaEventSynchronize(cudaEvent_t) { return cudaSuccess; }
static inline cudaError_t cudaEventElapsedTime(float* ms, cudaEvent_t, cudaEvent_t) { *ms = 0.001f; return cudaSuccess; }
static inline cudaError_t cudaPointerGetAttributes(cudaPointerAttributes* a, const void*) { a->type = cudaMemoryTypeUnregistered; return cudaSuccess; }
static inline cudaError_t cudaStreamBeginCapture(cudaStream_t, cudaStreamCaptureMode) { fake_cuda_capturing = 1; return cudaSuccess; }
static inline cudaError_t cudaStreamEndCapture(cudaStream_t, cudaGraph_t* g) { fake_cuda_capturing = 0; *g = (cudaGraph_t)malloc(8); return cudaSuccess; }
static inline cudaError_t cudaGraphInstantiate(cudaGraphExec_t* x, cudaGraph_t, unsigned long long) { *x = (cudaGraphExec_t)malloc(8); return cudaSuccess; }
static inline cudaError_t cudaGraphLaunch(cudaGraphExec_t, cudaStream_t) { return cudaSuccess; }
static inline cudaError_t cudaGraphDestroy(cudaGraph_t g) { free(g); return cudaSuccess; }
static inline cudaError_t cudaGraphExecDestroy(cudaGraphExec_t x) { free(x); return cudaSuccess; }
