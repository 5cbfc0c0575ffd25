/* TEST INFRASTRUCTURE ONLY -- host stand-ins for the few CUDA runtime calls that the reference's
 * CPU test harness makes (tensor.h:28, :38, :49, :74-93; cuda_timer.h:12-43; common.h:36-49), so
 * that its CPU attention can run on a machine without a GPU.  "Device" memory is host memory. */
#include <stdlib.h>
#include <string.h>

typedef int cudaError_t;
typedef void *cudaStream_t;
typedef void *cudaEvent_t;

cudaError_t cudaMalloc(void **p, size_t n) { *p = malloc(n ? n : 1); return *p ? 0 : 2; }
cudaError_t cudaFree(void *p) { free(p); return 0; }
cudaError_t cudaMemcpy(void *d, const void *s, size_t n, int kind) { (void)kind; memmove(d, s, n); return 0; }
cudaError_t cudaMemset(void *d, int v, size_t n) { memset(d, v, n); return 0; }
cudaError_t cudaEventCreate(cudaEvent_t *e) { *e = malloc(1); return 0; }
cudaError_t cudaEventDestroy(cudaEvent_t e) { free(e); return 0; }
cudaError_t cudaEventRecord(cudaEvent_t e, cudaStream_t s) { (void)e; (void)s; return 0; }
cudaError_t cudaEventSynchronize(cudaEvent_t e) { (void)e; return 0; }
cudaError_t cudaEventElapsedTime(float *ms, cudaEvent_t a, cudaEvent_t b) { (void)a; (void)b; *ms = 0.0f; return 0; }
const char *cudaGetErrorName(cudaError_t e) { (void)e; return "fake_cudart"; }
cudaError_t cudaRuntimeGetVersion(int *v) { *v = 0; return 0; }
cudaError_t cudaDriverGetVersion(int *v) { *v = 0; return 0; }
