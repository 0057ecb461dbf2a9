// Contract tests of the C++ host mirror (include/rwkv7_b200.hpp), runnable
// without a GPU: every case is rejected by the input checks before any CUDA
// call.  They restate the reference's panic tests: wkv7 T = 15
// (wkv7/mod.rs:329-336), mix6 wrong scale shape (mix6/mod.rs:248-257),
// token_shift_diff ShapeMismatch (token_shift_diff/mod.rs:330-347).
#include <cstdio>
#include <cstring>
#include <string>

#include "rwkv7_b200.hpp"

using namespace rwkv7b200;

static int failures = 0;
static float dummy[4096];

template <typename F>
static void expect_error(const char *what, const char *kind, const char *needle, F &&fn) {
    try {
        fn();
        std::printf("FAIL %s: no exception\n", what);
        ++failures;
    } catch (const KernelInputsError &e) {
        const bool ok = std::strcmp(e.kind(), kind) == 0 && std::strstr(e.what(), needle) != nullptr;
        if (!ok) {
            std::printf("FAIL %s: kind=%s message=%s\n", what, e.kind(), e.what());
            ++failures;
        } else {
            std::printf("ok   %s\n", what);
        }
    }
}

static TensorView f32(std::initializer_list<int64_t> shape) { return TensorView(dummy, RWKV7_F32, 0, shape); }

static Wkv7PretrainForwardInputs seq(std::initializer_list<int64_t> shape) {
    Wkv7PretrainForwardInputs in;
    in.receptance = in.weight_decay = in.replacement_key = in.value = in.removal_key_normalized = in.replacement =
        f32(shape);
    return in;
}

int main() {
    if (rwkv7_abi_version() != RWKV7_ABI_VERSION) {
        std::printf("FAIL abi version\n");
        return 1;
    }
    {
        auto in = seq({1, 15, 1, 4});
        auto y = f32({1, 15, 1, 4});
        expect_error("wkv7 forward_panics_on_wrong_context_len", "BadChunk", "multiple of chunk_len",
                     [&] { wkv7_pretrain_custom(in, y); });
    }
    {
        auto in = seq({2, 16, 2, 8});
        in.value = f32({2, 16, 2, 4});
        auto y = f32({2, 16, 2, 8});
        expect_error("wkv7 value shape", "ShapeMismatch", "value", [&] { wkv7_pretrain_custom(in, y); });
    }
    {
        Wkv7StatepassForwardInputs in{f32({2, 2, 8, 4}), seq({2, 16, 2, 8})};
        Wkv7StatepassForwardOutput out{f32({2, 16, 2, 8}), f32({2, 2, 8, 8})};
        expect_error("wkv7 initial_state shape", "ShapeMismatch", "initial_state",
                     [&] { wkv7_statepass_custom(in, out); });
    }
    {
        Mix6ForwardInputs in;
        in.embedded_context = f32({2, 4, 8});
        for (auto &s : in.scales) s = f32({1, 1, 8});
        in.scales[5] = f32({1, 1, 7});
        Mix6ForwardOutput out;
        for (auto &o : out.inputs) o = f32({2, 4, 8});
        expect_error("mix6 forward_panics_on_wrong_scale_shape", "ShapeMismatch", "gate_scale",
                     [&] { mix6_custom(in, out); });
    }
    {
        auto base = f32({2, 8, 32}), diff = f32({2, 8, 16}), scale = f32({1, 1, 32}), out = f32({2, 8, 32});
        expect_error("addcmul diff shape", "ShapeMismatch", "diff", [&] { addcmul_custom(base, diff, scale, out); });
    }
    {
        auto x = f32({2, 4, 8}), state = f32({3, 7}), diff = f32({2, 4, 8});
        TensorView ids(dummy, RWKV7_I32, 0, {2});
        expect_error("token_shift_diff shape_mismatch_panics", "ShapeMismatch", "embedded_token_shift",
                     [&] { token_shift_diff_custom(x, state, ids, diff); });
    }
    {   // training: snapshots of the wrong shape, and a backward workspace that is too small
        Wkv7StatepassForwardInputs in{TensorView(), seq({1, 32, 1, 8})};
        Wkv7SavedForward saved{f32({1, 32, 1, 8}), TensorView(), f32({1, 1, 3, 8, 8}), f32({1, 32, 1, 8})};
        expect_error("wkv7 forward_saved snapshots shape", "ShapeMismatch", "snapshots",
                     [&] { wkv7_forward_saved(in, saved); });
        saved.snapshots = f32({1, 1, 2, 8, 8});
        auto dy = f32({1, 32, 1, 8});
        Wkv7BackwardOutputs out{f32({1, 32, 1, 8}), f32({1, 32, 1, 8}), f32({1, 32, 1, 8}), f32({1, 32, 1, 4}),
                                f32({1, 32, 1, 8}), f32({1, 32, 1, 8}), TensorView()};
        expect_error("wkv7 backward value_grad shape", "ShapeMismatch", "value_grad",
                     [&] { wkv7_backward(in, saved, dy, TensorView(), out); });
        if (wkv7_backward_workspace_bytes(seq({2, 128, 2, 64})) == 0 || wkv7_backward_workspace_bytes(in.sequence) != 0) {
            std::printf("FAIL backward workspace size\n");
            ++failures;
        }
    }
    std::printf("%d failure(s)\n", failures);
    return failures ? 1 : 0;
}
