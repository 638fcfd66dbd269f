// Convolutions of NHWC bf16 tensors as implicit GEMMs on tcgen05 (see conv_tcgen05.cu): forward and input
// gradient for any small set of filter taps (3x3, strided 3x3, strided 1x1, the 4x4 space-to-depth stem), and
// the filter gradient as a split-K product over pixel patches.
#pragma once
#include <cuda_runtime.h>

namespace bfb {

constexpr int kConvMaxTaps = 16;

// One filter tap: the input pixel that meets output position (a, b) is (a * in_stride + dh, b * in_stride + dw);
// wt is the tap's slot in the filter tensor.
struct ConvTaps {
  int T;
  int dh[kConvMaxTaps];
  int dw[kConvMaxTaps];
  int wt[kConvMaxTaps];
};

// A dense 4-D view [n, h, w, c] of bf16 memory with explicit pitches in elements.  The pixel pitch may be
// smaller than c: the stem reads 64 consecutive values (4 pixels x 16 channels) per position of a
// 16-channel image, so that the four horizontal taps of its 4x4 filter are one reduction slice.
struct ConvView {
  const void* base;
  int n, h, w, c;
  long long pix_pitch, row_pitch, img_pitch;
};

// Patch of output positions one CTA owns: bn images x bh rows x bw columns, at most 128 positions.
// multiple_of_16: the patch has a multiple of 16 positions (the filter gradient reduces over positions in MMA
// steps of 16).  False when no such patch exists (W > 128, or no multiple of 16 within reach).
bool ConvPatch(int N, int H, int W, bool multiple_of_16, int* bw, int* bh, int* bn);

struct ConvProblem {
  ConvView x;            // x.c = reduction channels, a multiple of 64
  const void* w;         // filter_mode 0: [Cout, w_taps, x.c] (K-major B); 1: [x.c, w_taps, Cout] (MN-major B)
  int filter_mode;
  int w_taps;
  void* y;               // [N, Hy, Wy, Cout] dense NHWC
  int Hy, Wy, Cout;
  int Ho, Wo;            // grid of output positions (a, b); stored at (a * out_stride + out_ph, b * out_stride + out_pw)
  int out_stride, out_ph, out_pw;
  int in_stride;
  ConvTaps taps;
  float* col_stats;      // optional, 2 * Cout floats: += per-channel sum and sum of squares of the rounded output
};

bool ConvIgemmSupported(const ConvProblem& p);
// status: device word set to 1 when a bounded wait inside the kernel expired (may be null).
cudaError_t LaunchConvIgemm(const ConvProblem& p, unsigned int* status, cudaStream_t stream);

struct WgradProblem {
  ConvView dy;           // [N, Ho, Wo, Cout]; dense (pix_pitch == c)
  ConvView x;            // x.c = Cin, a multiple of 64
  int in_stride;
  ConvTaps taps;         // wt = slot of the tap in dw
  int w_taps;
  void* dw;              // bf16 [Cout, w_taps, x.c]
  // Scratch shared by every call on a stream: fp32 partial sums [Cout * w_taps * x.c] and one counter per output
  // tile.  Both must be zero on entry and are left zero on exit (the CTA that finishes a tile last converts it
  // and clears its words), so one zero-initialised allocation serves all layers.
  float* workspace;
  long long workspace_floats;
  unsigned int* counters;
  int n_counters;
};

bool ConvWgradSupported(const WgradProblem& p);
cudaError_t LaunchConvWgrad(const WgradProblem& p, unsigned int* status, cudaStream_t stream);

// 3x3 / stride 1 / pad 1 on the general kernel (kept for callers that only need this form).
bool Conv3x3Supported(int N, int H, int W, int Cin, int Cout);
// flip_taps: use filter tap (2 - r, 2 - s) for input tap (r, s) (the 180-degree rotation of the input-gradient form).
// filter_mode 0: w is [Cout,3,3,Cin].  1: w is [Cin,3,3,Cout] (the filter of the forward pass when this call
// computes an input gradient; Cin, Cout are this call's reduction and output channels), read as an MN-major operand.
cudaError_t LaunchConv3x3Nhwc(const void* x, const void* w, void* y, int N, int H, int W, int Cin, int Cout,
                              int flip_taps, int filter_mode, unsigned int* status, cudaStream_t stream);

}  // namespace bfb
