// Optimizer update rules as scalar host/device functors.
//
// Parity: the reference leaves the update rule to the user's store_push_value / init_store_value
// overrides (pico-ps/operator/SparsePushOperator.h:433-448; its tests use an integer sum/count,
// pico-ps/test/TestOps.h:87-118). This build ships the concrete rules a CTR / LLM trainer needs
// (SGD, Adagrad, FTRL-proximal, Adam/AdamW) plus SUM (value += push, the test operator) and SET
// (value = push, the DirectPush overwrite used by load / reshard / restore,
// pico-ps/operator/SparsePushOperator.h:520-574). The same code runs in the CPU oracle and in the
// kernels; device code uses the non-contracting intrinsics so both sides round identically.
#pragma once
#include <cmath>
#include <cstdint>

#include "../common/hash.h"

namespace psb {

enum OptType : int32_t {
    OPT_SGD = 0,
    OPT_ADAGRAD = 1,
    OPT_FTRL = 2,
    OPT_ADAM = 3,
    OPT_SUM = 4,
    OPT_SET = 5,
};

struct OptConfig {
    int32_t type = OPT_SGD;
    float lr = 0.01f;
    float eps = 1e-8f;
    float l1 = 0.f;       // FTRL
    float l2 = 0.f;       // FTRL
    float alpha = 0.05f;  // FTRL learning-rate scale
    float beta = 1.0f;    // FTRL
    float beta1 = 0.9f;   // Adam
    float beta2 = 0.999f;
    float weight_decay = 0.f;  // decoupled (AdamW / SGD)
    float bias_corr1 = 1.f;    // 1 - beta1^t, set by the host per step
    float bias_corr2 = 1.f;    // 1 - beta2^t
    float slot_init0 = 0.f;    // initial value of optimizer slot 0 (Adagrad accumulator, FTRL z, Adam m)
    float slot_init1 = 0.f;    // initial value of optimizer slot 1 (FTRL n, Adam v)
    int32_t step_from_epoch = 0;  // 1: kernels derive the Adam bias corrections from their own call counter
                                  // (needed when the launch is replayed from a CUDA graph)
};

// Adam bias corrections for (1-based) step t.
PSB_HD void opt_set_step(OptConfig& c, unsigned t) {
    if (c.type == OPT_ADAM) {
        c.bias_corr1 = 1.f - powf(c.beta1, (float)t);
        c.bias_corr2 = 1.f - powf(c.beta2, (float)t);
    }
}

PSB_HD int opt_num_slots(int type) {
    switch (type) {
        case OPT_ADAGRAD: return 1;
        case OPT_FTRL: return 2;
        case OPT_ADAM: return 2;
        default: return 0;
    }
}

#if defined(__CUDA_ARCH__)
#define PSB_MUL(a, b) __fmul_rn((a), (b))
#define PSB_ADD(a, b) __fadd_rn((a), (b))
#define PSB_SUB(a, b) __fsub_rn((a), (b))
#define PSB_DIV(a, b) __fdiv_rn((a), (b))
#define PSB_SQRT(a) __fsqrt_rn((a))
#else
#define PSB_MUL(a, b) ((a) * (b))
#define PSB_ADD(a, b) ((a) + (b))
#define PSB_SUB(a, b) ((a) - (b))
#define PSB_DIV(a, b) ((a) / (b))
#define PSB_SQRT(a) sqrtf((a))
#endif

// One coordinate: weight w, slots s0/s1, incoming (merged) push value g. kOpt >= 0 fixes the update rule at compile
// time (the caller vouches that c.type == kOpt): a kernel that inlines this four times per row then carries one
// rule's code instead of all of them.
template <int kOpt = -1>
PSB_HD void opt_update(const OptConfig& c, float& w, float& s0, float& s1, float g) {
    switch (kOpt >= 0 ? kOpt : c.type) {
        case OPT_SGD: {
            if (c.weight_decay != 0.f) w = PSB_SUB(w, PSB_MUL(PSB_MUL(c.lr, c.weight_decay), w));
            w = PSB_SUB(w, PSB_MUL(c.lr, g));
            break;
        }
        case OPT_ADAGRAD: {
            s0 = PSB_ADD(s0, PSB_MUL(g, g));
            w = PSB_SUB(w, PSB_DIV(PSB_MUL(c.lr, g), PSB_ADD(PSB_SQRT(s0), c.eps)));
            break;
        }
        case OPT_FTRL: {
            // s0 = z, s1 = n
            float n_new = PSB_ADD(s1, PSB_MUL(g, g));
            float sigma = PSB_DIV(PSB_SUB(PSB_SQRT(n_new), PSB_SQRT(s1)), c.alpha);
            s0 = PSB_SUB(PSB_ADD(s0, g), PSB_MUL(sigma, w));
            s1 = n_new;
            float az = fabsf(s0);
            if (az <= c.l1) {
                w = 0.f;
            } else {
                float sgn = s0 > 0.f ? 1.f : -1.f;
                float denom = PSB_ADD(PSB_DIV(PSB_ADD(c.beta, PSB_SQRT(s1)), c.alpha), c.l2);
                w = PSB_DIV(PSB_SUB(PSB_MUL(sgn, c.l1), s0), denom);
            }
            break;
        }
        case OPT_ADAM: {
            s0 = PSB_ADD(PSB_MUL(c.beta1, s0), PSB_MUL(PSB_SUB(1.f, c.beta1), g));
            s1 = PSB_ADD(PSB_MUL(c.beta2, s1), PSB_MUL(PSB_SUB(1.f, c.beta2), PSB_MUL(g, g)));
            float mhat = PSB_DIV(s0, c.bias_corr1);
            float vhat = PSB_DIV(s1, c.bias_corr2);
            if (c.weight_decay != 0.f) w = PSB_SUB(w, PSB_MUL(PSB_MUL(c.lr, c.weight_decay), w));
            w = PSB_SUB(w, PSB_DIV(PSB_MUL(c.lr, mhat), PSB_ADD(PSB_SQRT(vhat), c.eps)));
            break;
        }
        case OPT_SUM: {
            w = PSB_ADD(w, g);
            break;
        }
        case OPT_SET: {
            w = g;
            break;
        }
        default: break;
    }
}

}  // namespace psb
