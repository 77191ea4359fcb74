/*
 * Drives a CVM runtime library the way the reference's Go package does: through the dlopen shim of
 * kernel/dlopen.h (plugin_open with RTLD_NOW|RTLD_GLOBAL, one dlsym per call behind the
 * dl_CVMAPI* wrappers) in the call order of kernel/libcvm.go:57-133 and kernel/model.go:102-133:
 * LoadModel, the length / type-size / storage / gas queries, GetVersion and GetPreprocessMethod
 * into 34-byte buffers, Inference into a caller buffer of GetOutputLength bytes, FreeModel.
 *
 * The header is NOT part of this repository: the program is compiled with -I<reference>/kernel
 * against the reference checkout (see build_caller() in tests/test_caller_shim.py).
 *
 *   go_shim_caller <library.so> <graph.json> <params.bin> <input.bin> <output.bin> <device_type> <device_id>
 *
 * Prints "@key=value" tokens with every status and query result (the reference library writes lines
 * of its own to stdout in between); exit code 0 when every call returned SUCCEED.
 */
#include "dlopen.h"
#include <string.h>

static char* read_file(const char* path, long* len) {
  FILE* f = fopen(path, "rb");
  if (!f) { fprintf(stderr, "cannot open %s\n", path); exit(3); }
  fseek(f, 0, SEEK_END);
  *len = ftell(f);
  fseek(f, 0, SEEK_SET);
  char* buf = (char*)malloc((size_t)*len + 1);
  if (fread(buf, 1, (size_t)*len, f) != (size_t)*len) { fprintf(stderr, "short read on %s\n", path); exit(3); }
  buf[*len] = 0;
  fclose(f);
  return buf;
}

int main(int argc, char** argv) {
  if (argc != 8) { fprintf(stderr, "usage: %s lib json params input output device_type device_id\n", argv[0]); return 2; }
  char* err = NULL;
  void* lib = plugin_open(argv[1], &err);
  if (!lib) { fprintf(stderr, "plugin_open failed: %s\n", err ? err : "?"); return 4; }
  long jlen, plen, ilen;
  char* json = read_file(argv[2], &jlen);
  char* params = read_file(argv[3], &plen);
  char* input = read_file(argv[4], &ilen);
  void* net = NULL;
  int worst = 0, st;
  st = dl_CVMAPILoadModel(lib, json, (int)jlen, params, (int)plen, &net, atoi(argv[6]), atoi(argv[7]));
  printf("@load=%d ", st);
  if (st != SUCCEED) { printf("\n"); return 10 + st; }
  unsigned long long in_len = 0, out_len = 0, in_ts = 0, out_ts = 0, storage = 0, gas = 0, gas_file = 0;
  st = dl_CVMAPIGetInputLength(lib, net, &in_len); worst |= st; printf("@input_length=%llu ", in_len);
  st = dl_CVMAPIGetOutputLength(lib, net, &out_len); worst |= st; printf("@output_length=%llu ", out_len);
  st = dl_CVMAPIGetInputTypeSize(lib, net, &in_ts); worst |= st; printf("@input_type_size=%llu ", in_ts);
  st = dl_CVMAPIGetOutputTypeSize(lib, net, &out_ts); worst |= st; printf("@output_type_size=%llu ", out_ts);
  st = dl_CVMAPIGetStorageSize(lib, net, &storage); worst |= st; printf("@storage=%llu ", storage);
  st = dl_CVMAPIGetGasFromModel(lib, net, &gas); printf("@gas_status=%d @gas=%llu ", st, gas);
  char version[34], method[34];
  memset(version, 0, sizeof(version));
  memset(method, 0, sizeof(method));
  st = dl_CVMAPIGetVersion(lib, net, version); worst |= st;
  st = dl_CVMAPIGetPreprocessMethod(lib, net, method); worst |= st;
  printf("@version=[%s] @method=[%s] ", version, method);
  if ((unsigned long long)ilen != in_len) { fprintf(stderr, "input file has %ld bytes, the model wants %llu\n", ilen, in_len); return 5; }
  char* out = (char*)calloc((size_t)out_len + 1, 1);
  /* two inferences in a row on one handle, as a node that validates several blocks does */
  st = dl_CVMAPIInference(lib, net, input, (int)ilen, out); worst |= st; printf("@infer=%d ", st);
  st = dl_CVMAPIInference(lib, net, input, (int)ilen, out); worst |= st; printf("@infer2=%d ", st);
  FILE* f = fopen(argv[5], "wb");
  if (!f || fwrite(out, 1, (size_t)out_len, f) != (size_t)out_len) { fprintf(stderr, "cannot write %s\n", argv[5]); return 6; }
  fclose(f);
  st = dl_CVMAPIGetGasFromGraphFile(lib, json, &gas_file); printf("@gas_file_status=%d @gas_file=%llu ", st, gas_file);
  st = dl_CVMAPIFreeModel(lib, net); worst |= st; printf("@free=%d\n", st);
  return worst == SUCCEED ? 0 : 20 + worst;
}
