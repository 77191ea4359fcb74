/* Host-side functions of the kernel C-ABI that need no device: the shapes the tensor-core
 * convolution cuts along K and the scratch they want, and the operand order the stem convolution
 * packs its filter into.  Compiled as plain C against include/cvmk_kernels.h (which is therefore
 * checked to be a C header) and linked with the runtime library; the test reads the lines printed
 * here and the packed bytes written to the file named on the command line.
 *
 *   host_fns workspace N H W C OC KH KW        -> "@supported=.. @workspace=.."
 *   host_fns grouped N H W C groups K stride   -> "@supported=.." (OC = C, padding K / 2)
 *   host_fns stem N H W C OC KH KW stride pad out.bin
 *                                              -> "@supported=.. @weight_bytes=.. @pack=.."
 * The stem filter is w[oc][c][ky][kx] = ((oc * 131 + c * 31 + ky * 7 + kx) mod 255) - 127.
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "cvmk_kernels.h"

static int arg(char** argv, int i) { return atoi(argv[i]); }

int main(int argc, char** argv) {
  if (argc >= 9 && strcmp(argv[1], "workspace") == 0) {
    cvmk_conv_desc d;
    memset(&d, 0, sizeof(d));
    d.y_dtype = CVMK_I8;
    d.N = arg(argv, 2); d.H = arg(argv, 3); d.W = arg(argv, 4); d.C = arg(argv, 5);
    d.OC = arg(argv, 6); d.KH = arg(argv, 7); d.KW = arg(argv, 8);
    d.stride_h = d.stride_w = 1; d.dil_h = d.dil_w = 1;
    d.pad_h = d.KH / 2; d.pad_w = d.KW / 2;
    d.OH = d.H; d.OW = d.W;
    printf("@supported=%d @workspace=%lld\n", cvmk_conv2d_tc_supported(&d), (long long)cvmk_conv2d_tc_workspace_bytes(&d));
    return 0;
  }
  if (argc >= 9 && strcmp(argv[1], "grouped") == 0) {
    cvmk_conv_desc d;
    memset(&d, 0, sizeof(d));
    d.y_dtype = CVMK_I8;
    d.N = arg(argv, 2); d.H = arg(argv, 3); d.W = arg(argv, 4); d.C = d.OC = arg(argv, 5);
    d.groups = arg(argv, 6);
    d.KH = d.KW = arg(argv, 7);
    d.stride_h = d.stride_w = arg(argv, 8); d.dil_h = d.dil_w = 1;
    d.pad_h = d.pad_w = d.KH / 2;
    d.OH = (d.H + 2 * d.pad_h - d.KH) / d.stride_h + 1;
    d.OW = (d.W + 2 * d.pad_w - d.KW) / d.stride_w + 1;
    printf("@supported=%d\n", cvmk_conv2d_tc_supported(&d));
    return 0;
  }
  if (argc >= 12 && strcmp(argv[1], "stem") == 0) {
    cvmk_stem_conv_desc d;
    memset(&d, 0, sizeof(d));
    d.N = arg(argv, 2); d.H = arg(argv, 3); d.W = arg(argv, 4); d.C = arg(argv, 5);
    d.OC = arg(argv, 6); d.KH = arg(argv, 7); d.KW = arg(argv, 8);
    d.stride_h = d.stride_w = arg(argv, 9);
    d.pad_h = d.pad_w = arg(argv, 10);
    d.clamp = 127;
    d.OH = (d.H + 2 * d.pad_h - d.KH) / d.stride_h + 1;
    d.OW = (d.W + 2 * d.pad_w - d.KW) / d.stride_w + 1;
    const int ok = cvmk_conv2d_stem_supported(&d);
    const long long bytes = (long long)cvmk_conv2d_stem_weight_bytes(&d);
    int rc = -1;
    if (ok && bytes > 0) {
      const size_t n = (size_t)d.OC * d.C * d.KH * d.KW;
      int32_t* w = (int32_t*)malloc(n * sizeof(int32_t));
      int8_t* packed = (int8_t*)malloc((size_t)bytes);
      size_t at = 0;
      for (int oc = 0; oc < d.OC; ++oc)
        for (int c = 0; c < d.C; ++c)
          for (int ky = 0; ky < d.KH; ++ky)
            for (int kx = 0; kx < d.KW; ++kx) w[at++] = (oc * 131 + c * 31 + ky * 7 + kx) % 255 - 127;
      memset(packed, 0x5a, (size_t)bytes);
      rc = cvmk_conv2d_stem_pack_weights(&d, w, packed);
      FILE* f = fopen(argv[11], "wb");
      if (!f || fwrite(packed, 1, (size_t)bytes, f) != (size_t)bytes) rc = -2;
      if (f) fclose(f);
      free(w); free(packed);
    }
    printf("@supported=%d @weight_bytes=%lld @pack=%d\n", ok, bytes, rc);
    return 0;
  }
  fprintf(stderr, "usage: host_fns workspace|stem ...\n");
  return 2;
}
