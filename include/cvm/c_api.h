/*
 * C-ABI of libcvm_runtime.so: the twelve entry points that the reference declares in
 * kernel/c_api.h:30-49 (identical copy: include/cvm/c_api.h:33-52) and implements in
 * src/core/c_api.cc.  The Go binding dlopen()s the library and dlsym()s these names on every call
 * (kernel/dlopen.h:11-17,47-78); Python binds them through ctypes
 * (python/cvm/_ctypes/runtime.py:12-159).  Names, argument meaning, ownership and status codes
 * are the reference's; the operator kernels behind them run on one NVIDIA B200 (sm_100a).
 *
 * Status: SUCCEED (0); ERROR_LOGIC (1) when the model or the input is at fault (every VERIFY of the
 * reference); ERROR_RUNTIME (2) for everything else (null arguments, CUDA failures, malformed
 * JSON, unknown operators or attributes).  A line "ERROR: <text>" is printed to stdout on failure,
 * as include/cvm/errors.h:15-36 does.  No exception crosses this boundary.
 */
#ifndef CVM_C_API_H_
#define CVM_C_API_H_

#define CVM_DLL __attribute__((visibility("default")))

#ifdef __cplusplus
extern "C" {
#endif

enum { SUCCEED = 0, ERROR_LOGIC = 1, ERROR_RUNTIME = 2 };

/* src/core/c_api.cc:22-43.  graph_json / param_bytes are copied.  device_type follows the
 * reference's numbering (0 CPU, 1 GPU, 2 FORMAL); this library implements 1 only and answers
 * ERROR_RUNTIME for 0 and 2 (there is no CPU path), ERROR_RUNTIME for anything else like the
 * reference.  device_id selects the GPU.  On success *net owns the model until CVMAPIFreeModel. */
CVM_DLL int CVMAPILoadModel(const char* graph_json, int graph_strlen, const char* param_bytes,
                            int param_strlen, void** net, int device_type, int device_id);
/* src/core/c_api.cc:46-51 */
CVM_DLL int CVMAPIFreeModel(void* net);
/* src/core/c_api.cc:53-77.  input_len must equal CVMAPIGetInputLength(); output_data must hold
 * CVMAPIGetOutputLength() bytes.  One handle must not be used from two threads at once. */
CVM_DLL int CVMAPIInference(void* net, char* input_data, int input_len, char* output_data);

/* src/core/c_api.cc:79-95.  Buffers of at least 33 bytes; GetPreprocessMethod returns the graph's
 * "postprocess" key, as in the reference. */
CVM_DLL int CVMAPIGetVersion(void* net, char* version);
CVM_DLL int CVMAPIGetPreprocessMethod(void* net, char* method);

/* src/core/c_api.cc:97-127, src/core/model.cc:293-335 */
CVM_DLL int CVMAPIGetInputLength(void* net, unsigned long long* size);
CVM_DLL int CVMAPIGetOutputLength(void* net, unsigned long long* size);
CVM_DLL int CVMAPIGetInputTypeSize(void* net, unsigned long long* size);
CVM_DLL int CVMAPIGetOutputTypeSize(void* net, unsigned long long* size);

/* src/core/c_api.cc:129-152.  Storage size is the reference's int32 pool figure
 * (src/runtime/graph_runtime.cc:565-574); gas is CvmRuntime::GetOps
 * (src/runtime/infer_attr.cc:93-159).  GetGasFromGraphFile takes a NUL-terminated string. */
CVM_DLL int CVMAPIGetStorageSize(void* net, unsigned long long* gas);
CVM_DLL int CVMAPIGetGasFromModel(void* net, unsigned long long* gas);
CVM_DLL int CVMAPIGetGasFromGraphFile(const char* graph_json, unsigned long long* gas);

#ifdef __cplusplus
}
#endif
#endif /* CVM_C_API_H_ */
