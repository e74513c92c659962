// Activation functions of the Gate / Activation modules and their derivatives (codes shared by the host tables,
// the elementwise kernels and the gated epilogue of the dense contraction).
#pragma once
#include <cuda_runtime.h>

namespace e3b {

enum GateAct { kGSilu = 0, kGTanh = 1, kGRelu = 2, kGIdentity = 3, kGSigmoid = 4, kGAbs = 5 };

__device__ __forceinline__ float gate_act(int kind, float x) {
    switch (kind) {
        case kGSilu: return x / (1.0f + expf(-x));
        case kGTanh: return tanhf(x);
        case kGRelu: return fmaxf(x, 0.0f);
        case kGSigmoid: return 1.0f / (1.0f + expf(-x));
        case kGAbs: return fabsf(x);
        default: return x;
    }
}
__device__ __forceinline__ float gate_act_grad(int kind, float x) {
    switch (kind) {
        case kGSilu: {
            const float s = 1.0f / (1.0f + expf(-x));
            return s * (1.0f + x * (1.0f - s));
        }
        case kGTanh: {
            const float t = tanhf(x);
            return 1.0f - t * t;
        }
        case kGRelu: return x > 0.0f ? 1.0f : 0.0f;
        case kGSigmoid: {
            const float s = 1.0f / (1.0f + expf(-x));
            return s * (1.0f - s);
        }
        case kGAbs: return x > 0.0f ? 1.0f : (x < 0.0f ? -1.0f : 0.0f);
        default: return 1.0f;
    }
}

}  // namespace e3b
