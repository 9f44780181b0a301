// A stand-in for the CUDA runtime, for running the NVLINK backend's HOST code on a machine without a GPU.
//
// "Device memory" is host memory, a stream is a thread that runs queued tasks in order, an event is a marker in a
// stream, the copy kernels are functions that run as such tasks (fake_xfer_kernels.cpp).  What the backend's host side
// relies on is modelled; nothing else: stream order, events and stream waits, asynchronous copies (a copy from
// pageable host memory takes its source at once, a copy from pinned memory when it runs), pinned and registered host
// ranges, per-device allocations with pointer attributes, peer access, IPC handles (device memory is a shared-memory
// object that another process maps), the driver's virtual-memory calls (export of an allocation as a file descriptor,
// import, reserve / map / unmap), "not ready" as the last error.
//
// Only the test build of the plug-in sees this header (it shadows the real <cuda_runtime.h> on the include path).
#ifndef NIXL_B200_FAKE_CUDA_RUNTIME_H
#define NIXL_B200_FAKE_CUDA_RUNTIME_H

#include <cstddef>
#include <cstdint>

#ifndef __host__
#define __host__
#endif
#ifndef __device__
#define __device__
#endif

extern "C" {

typedef enum cudaError {
    cudaSuccess = 0,
    cudaErrorInvalidValue = 1,
    cudaErrorMemoryAllocation = 2,
    cudaErrorInvalidDevice = 101,
    cudaErrorInvalidResourceHandle = 400,
    cudaErrorNotReady = 600,
    cudaErrorPeerAccessAlreadyEnabled = 704,
    cudaErrorHostMemoryAlreadyRegistered = 712,
    cudaErrorHostMemoryNotRegistered = 713,
    cudaErrorNotSupported = 801,
    cudaErrorUnknown = 999
} cudaError_t;

struct FakeCudaStream;
struct FakeCudaEvent;
typedef FakeCudaStream *cudaStream_t;
typedef FakeCudaEvent *cudaEvent_t;

typedef struct cudaIpcMemHandle_st {
    char reserved[64];
} cudaIpcMemHandle_t;

typedef struct cudaUUID_st {
    char bytes[16];
} cudaUUID_t;

struct cudaDeviceProp {
    char name[256];
    cudaUUID_t uuid;
    size_t totalGlobalMem;
    int multiProcessorCount;
    int major, minor;
    int pciBusID, pciDeviceID, pciDomainID;
};

enum cudaMemoryType { cudaMemoryTypeUnregistered = 0, cudaMemoryTypeHost = 1, cudaMemoryTypeDevice = 2, cudaMemoryTypeManaged = 3 };
struct cudaPointerAttributes {
    enum cudaMemoryType type;
    int device;
    void *devicePointer;
    void *hostPointer;
};

enum cudaMemcpyKind { cudaMemcpyHostToHost = 0, cudaMemcpyHostToDevice = 1, cudaMemcpyDeviceToHost = 2, cudaMemcpyDeviceToDevice = 3, cudaMemcpyDefault = 4 };
enum cudaDeviceAttr { cudaDevAttrMultiProcessorCount = 16 };
enum cudaDriverEntryPointQueryResult { cudaDriverEntryPointSuccess = 0, cudaDriverEntryPointSymbolNotFound = 1, cudaDriverEntryPointVersionNotSufficent = 2 };

#define cudaStreamDefault 0x00u
#define cudaStreamNonBlocking 0x01u
#define cudaEventDefault 0x00u
#define cudaEventDisableTiming 0x02u
#define cudaHostAllocDefault 0x00u
#define cudaHostAllocPortable 0x01u
#define cudaHostAllocMapped 0x02u
#define cudaHostRegisterDefault 0x00u
#define cudaHostRegisterPortable 0x01u
#define cudaHostRegisterMapped 0x02u
#define cudaIpcMemLazyEnablePeerAccess 0x01u
#define cudaEnableDefault 0x0ull

cudaError_t cudaGetLastError(void);
cudaError_t cudaPeekAtLastError(void);
const char *cudaGetErrorString(cudaError_t e);

cudaError_t cudaGetDeviceCount(int *count);
cudaError_t cudaGetDevice(int *device);
cudaError_t cudaSetDevice(int device);
cudaError_t cudaDeviceGetAttribute(int *value, enum cudaDeviceAttr attr, int device);
cudaError_t cudaGetDeviceProperties(struct cudaDeviceProp *prop, int device);
cudaError_t cudaDeviceSynchronize(void);
cudaError_t cudaDeviceCanAccessPeer(int *can, int device, int peer);
cudaError_t cudaDeviceEnablePeerAccess(int peer, unsigned int flags);

cudaError_t cudaMalloc(void **ptr, size_t size);
cudaError_t cudaFree(void *ptr);
cudaError_t cudaHostAlloc(void **ptr, size_t size, unsigned int flags);
cudaError_t cudaFreeHost(void *ptr);
cudaError_t cudaHostRegister(void *ptr, size_t size, unsigned int flags);
cudaError_t cudaHostUnregister(void *ptr);
cudaError_t cudaHostGetDevicePointer(void **dev, void *host, unsigned int flags);
cudaError_t cudaPointerGetAttributes(struct cudaPointerAttributes *attr, const void *ptr);

cudaError_t cudaMemset(void *ptr, int value, size_t count);
cudaError_t cudaMemcpy(void *dst, const void *src, size_t count, enum cudaMemcpyKind kind);
cudaError_t cudaMemcpyAsync(void *dst, const void *src, size_t count, enum cudaMemcpyKind kind, cudaStream_t stream);

cudaError_t cudaStreamCreate(cudaStream_t *stream);
cudaError_t cudaStreamCreateWithFlags(cudaStream_t *stream, unsigned int flags);
cudaError_t cudaStreamDestroy(cudaStream_t stream);
cudaError_t cudaStreamSynchronize(cudaStream_t stream);
cudaError_t cudaStreamWaitEvent(cudaStream_t stream, cudaEvent_t event, unsigned int flags);

cudaError_t cudaEventCreate(cudaEvent_t *event);
cudaError_t cudaEventCreateWithFlags(cudaEvent_t *event, unsigned int flags);
cudaError_t cudaEventDestroy(cudaEvent_t event);
cudaError_t cudaEventRecord(cudaEvent_t event, cudaStream_t stream);
cudaError_t cudaEventQuery(cudaEvent_t event);
cudaError_t cudaEventSynchronize(cudaEvent_t event);

cudaError_t cudaIpcGetMemHandle(cudaIpcMemHandle_t *handle, void *ptr);
cudaError_t cudaIpcOpenMemHandle(void **ptr, cudaIpcMemHandle_t handle, unsigned int flags);
cudaError_t cudaIpcCloseMemHandle(void *ptr);

cudaError_t cudaGetDriverEntryPoint(const char *symbol, void **fn, unsigned long long flags, enum cudaDriverEntryPointQueryResult *result);

} // extern "C"

// ---- the stand-in's own interface (tests and the stand-in kernels) ----
#include <functional>

namespace fake_cuda {
// Queues `task` on `stream` (nullptr: the current device's default stream).
void enqueue(cudaStream_t stream, std::function<void()> task);
// Queues a task that holds the stream for `microseconds` (a long-running kernel in front of whatever comes next).
void enqueueDelay(cudaStream_t stream, unsigned microseconds);
// Number of devices the stand-in reports (environment FAKE_CUDA_DEVICES, default 2); tasks run so far.
int deviceCount();
uint64_t tasksRun();
// "Virtual memory management" allocations (what cuMemCreate + cuMemMap give: PyTorch's expandable segments, engines' own
// pools): `chunks` physical allocations of `chunk_bytes` mapped back to back into one address range of `device`.  CUDA
// IPC refuses such memory; it is shared through the driver's export / import calls, which the stand-in offers through
// cudaGetDriverEntryPoint.
void *mallocVmm(size_t chunk_bytes, int chunks, int device);
void freeVmm(void *ptr);
// Failure injection for the stand-in kernels: the next `count` launches of that kind fail with cudaErrorUnknown.
enum class LaunchKind { Copy = 0, Signal = 1, Proxy = 2 };
void failLaunches(LaunchKind kind, int count);
bool takeLaunchFailure(LaunchKind kind); // used by the stand-in kernels: true = fail this launch
} // namespace fake_cuda

#endif
