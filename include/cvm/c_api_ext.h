/*
 * Measurement helpers exported next to the reference C-ABI.  They have no counterpart in the
 * reference (whose only instrumentation is the compile-time PROFILE table,
 * src/runtime/graph_runtime.cc:62-87); benchmarks use them to time the kernels with the input
 * already resident in device memory and to attribute device time to operators.
 * Status codes are those of include/cvm/c_api.h.
 */
#ifndef CVM_C_API_EXT_H_
#define CVM_C_API_EXT_H_

#ifndef CVM_DLL
#define CVM_DLL __attribute__((visibility("default")))
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Text of the last error a CVMAPI* / CVMX* call returned on this thread (the reference only prints
 * it); valid until the next failing call of the thread. */
CVM_DLL const char* CVMXLastError(void);
/* Number of kernel launches one inference enqueues (fused operators count once). */
CVM_DLL int CVMXStepCount(void* net, unsigned long long* n);
/* Device memory held by the model: weights, activations, staging. */
CVM_DLL int CVMXDeviceBytes(void* net, unsigned long long* n);
/* Activation memory under the lifetime planner: `buffers` = the sizes of all planned activation
 * buffers added up (what one allocation per buffer would take), `physical` = the device memory
 * that backs them once buffers with disjoint lifetimes share it.  Both 0 when the planner is off. */
CVM_DLL int CVMXActivationBytes(void* net, unsigned long long* buffers, unsigned long long* physical);
/* Replays the model's kernels `iters` times on the input of the last CVMAPIInference call (no
 * upload, no download) and returns the elapsed device time, measured with CUDA events on the
 * model's stream, in milliseconds. */
CVM_DLL int CVMXReplayDevice(void* net, int iters, float* total_ms);
/* Runs one inference launch by launch with a CUDA event between launches and writes one line
 * "<operator label>\t<milliseconds>\n" per launch into `text` (NUL-terminated). */
CVM_DLL int CVMXProfileSteps(void* net, const char* input_data, int input_len, char* text,
                             int text_len);

/* Writes `code` into the model's device status word: the word every tensor-core kernel ORs a
 * non-zero value into when one of its bounded waits runs out.  The next CVMAPIInference on the
 * handle then answers ERROR_RUNTIME, clears the word and leaves the handle usable.  Exists so that
 * this error path can be exercised without making a kernel fail. */
CVM_DLL int CVMXSetStatusWord(void* net, int code);

#ifdef __cplusplus
}
#endif
#endif /* CVM_C_API_EXT_H_ */
