/* Link-time stand-ins for what the reference's matrix test program names but this
 * repository never runs.  TEST INFRASTRUCTURE ONLY.
 *
 * The reference test program that ref_wrap.cu includes also holds cases that read model
 * files and cases that drive a PTX module through the CUDA driver API.  Neither is called
 * through the binding layer, but their symbols must resolve when the library is loaded on a
 * machine that has no driver library and no model-file reader.  Every stand-in is weak and
 * reports failure, so a real definition wins wherever one is present. */
#include <stddef.h>
#include <stdint.h>

#define REF_WEAK __attribute__((weak))

REF_WEAK int aotx_modelfile_open(const char *path, void **file) { (void)path; (void)file; return 1; }
REF_WEAK void aotx_modelfile_close(void *file) { (void)file; }
REF_WEAK uint64_t aotx_modelfile_tensor_count(const void *file) { (void)file; return 0; }
REF_WEAK int aotx_modelfile_tensor(const void *file, uint64_t index, void *info) { (void)file; (void)index; (void)info; return 1; }
REF_WEAK int aotx_modelfile_find(const void *file, const char *name, void *info) { (void)file; (void)name; (void)info; return 1; }
REF_WEAK int aotx_modelfile_read(const void *file, uint64_t offset, uint64_t bytes, void *buffer) { (void)file; (void)offset; (void)bytes; (void)buffer; return 1; }

/* CUDA_ERROR_NOT_INITIALIZED */
#define REF_DRIVER_ABSENT 3
REF_WEAK int cuInit(unsigned int flags) { (void)flags; return REF_DRIVER_ABSENT; }
REF_WEAK int cuDeviceGet(int *device, int ordinal) { (void)device; (void)ordinal; return REF_DRIVER_ABSENT; }
REF_WEAK int cuDevicePrimaryCtxRetain(void **ctx, int device) { (void)ctx; (void)device; return REF_DRIVER_ABSENT; }
REF_WEAK int cuCtxSetCurrent(void *ctx) { (void)ctx; return REF_DRIVER_ABSENT; }
REF_WEAK int cuGetErrorName(int error, const char **name) { (void)error; *name = "driver absent"; return 0; }
REF_WEAK int cuModuleLoadData(void **module, const void *image) { (void)module; (void)image; return REF_DRIVER_ABSENT; }
REF_WEAK int cuModuleGetFunction(void **function, void *module, const char *name) { (void)function; (void)module; (void)name; return REF_DRIVER_ABSENT; }
REF_WEAK int cuModuleUnload(void *module) { (void)module; return REF_DRIVER_ABSENT; }
REF_WEAK int cuGraphCreate(void **graph, unsigned int flags) { (void)graph; (void)flags; return REF_DRIVER_ABSENT; }
REF_WEAK int cuGraphAddKernelNode_v2(void **node, void *graph, const void *deps, size_t count, const void *params) { (void)node; (void)graph; (void)deps; (void)count; (void)params; return REF_DRIVER_ABSENT; }
REF_WEAK int cuGraphInstantiateWithFlags(void **exec, void *graph, unsigned long long flags) { (void)exec; (void)graph; (void)flags; return REF_DRIVER_ABSENT; }
REF_WEAK int cuGraphLaunch(void *exec, void *stream) { (void)exec; (void)stream; return REF_DRIVER_ABSENT; }
REF_WEAK int cuGraphExecDestroy(void *exec) { (void)exec; return REF_DRIVER_ABSENT; }
REF_WEAK int cuGraphDestroy(void *graph) { (void)graph; return REF_DRIVER_ABSENT; }
