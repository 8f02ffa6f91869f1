// Scratch-reusing callers of the packed-int4 primitives: the second in-tree consumer of the same kernels.
//
// Mirrors vyre-self-substrate/src/math/quantized_dispatch.rs:30-90 and the six modules under quantized_dispatch/
// (unpack.rs, dot.rs, matvec.rs, batched_matvec.rs, batched_matmul.rs, top1.rs; shape rules in shapes.rs:12-76): each
// `*_via_with_scratch_into` validates the host slices against the shape (same conditions, same `Fix:` texts), takes the
// Program for that shape from a cache the caller owns, dispatches it with the inputs in slot order and checks that
// exactly the expected output bytes came back. There the dispatcher is a trait object and the scratch holds host
// staging vectors plus a Program cache per wrapper; here the dispatcher is a device of this library and ONE scratch
// object caches, per (wrapper, shape), the whole chain Program -> Artifact -> TargetPayload -> ArtifactInstance, so
// that a repeated call costs one submission and no compilation. Host staging is the submission's own pinned pool.
//
// DispatchError (vyre-self-substrate/src/optimizer/dispatcher.rs:100-120) maps onto three status codes whose messages
// carry the reference's Display prefix.
#include <array>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "model.hpp"

using namespace vyb;

struct vyb_quantized_scratch {
    struct Entry {
        vyb_program* program = nullptr;
        vyb_artifact* artifact = nullptr;
        vyb_payload* payload = nullptr;
        vyb_instance* instance = nullptr;
        uint8_t digest[32] = {};
        std::vector<vyb_buffer_decl> inputs;  // ReadOnly / ReadWrite values in slot order
        uint32_t output_id = 0;
        uint32_t outputs = 0;
    };
    vyb_device* device = nullptr;
    std::mutex mu;
    std::map<std::array<uint32_t, 4>, Entry> cache;
    uint64_t hits = 0, misses = 0;
    std::vector<uint8_t> zeros;  // the ReadWrite output of unpack_i4x8 is bound as zero bytes (unpack.rs:72)
};

namespace {

enum Wrapper : uint32_t { W_UNPACK = 1, W_DOT, W_MATVEC, W_BATCHED_MATVEC, W_BATCHED_MATMUL, W_TOP1 };

int32_t bad_inputs(const std::string& fix) { return fail(VYB_ERR_DISPATCH_BAD_INPUTS, "dispatcher input mismatch: " + fix); }
int32_t backend_error(const std::string& fix) { return fail(VYB_ERR_DISPATCH_BACKEND, "dispatcher backend error: " + fix); }
int32_t rejected() {
    // the failing call has left its BackendError text as the last error; keep it behind the dispatcher's prefix
    return fail(VYB_ERR_DISPATCH_REJECTED, std::string("dispatcher rejected program: ") + vyb_last_error_message());
}

void drop(vyb_quantized_scratch::Entry& e) {
    if (e.instance) vyb_instance_free(e.instance);
    if (e.payload) vyb_payload_free(e.payload);
    if (e.artifact) vyb_artifact_free(e.artifact);
    if (e.program) vyb_program_free(e.program);
    e = vyb_quantized_scratch::Entry();
}

// the cached chain for one (wrapper, shape); `build` makes the Program on a miss
template <class Build>
int32_t entry_for(vyb_quantized_scratch* s, const std::array<uint32_t, 4>& key, Build build,
                  vyb_quantized_scratch::Entry** out) {
    auto it = s->cache.find(key);
    if (it != s->cache.end()) {
        ++s->hits;
        *out = &it->second;
        return VYB_OK;
    }
    ++s->misses;
    if (!s->device)
        return fail(VYB_ERR_DISPATCH_REJECTED, "dispatcher rejected program: Fix: this scratch was made without a device; make it with the device that is to run the dispatch.");
    vyb_quantized_scratch::Entry e;
    if (build(&e.program) != VYB_OK) return rejected();
    if (vyb_program_is_trap(e.program)) {  // the builders return trap programs for shapes they refuse
        const std::string why = vyb_program_trap_message(e.program);
        drop(e);
        return fail(VYB_ERR_DISPATCH_REJECTED, "dispatcher rejected program: " + why);
    }
    if (vyb_compile(e.program, &e.artifact) != VYB_OK || vyb_target_compile(e.artifact, &e.payload) != VYB_OK ||
        vyb_materialize(s->device, e.artifact, e.payload, &e.instance) != VYB_OK) {
        const int32_t rc = rejected();
        drop(e);
        return rc;
    }
    vyb_artifact_digest(e.artifact, e.digest);
    const uint32_t n = vyb_program_buffer_count(e.program);
    for (uint32_t i = 0; i < n; ++i) {
        vyb_buffer_decl d;
        if (vyb_program_buffer(e.program, i, &d) != VYB_OK) continue;
        if (d.access == VYB_ACCESS_READ_ONLY || d.access == VYB_ACCESS_READ_WRITE) e.inputs.push_back(d);
        if (d.access == VYB_ACCESS_OUTPUT || d.access == VYB_ACCESS_READ_WRITE) {
            e.output_id = d.binding;
            ++e.outputs;
        }
    }
    auto placed = s->cache.emplace(key, e);
    *out = &placed.first->second;
    return VYB_OK;
}

// one dispatch: host inputs in slot order, exactly one output of `expected_bytes`, copied into `dst`
int32_t dispatch_into(vyb_quantized_scratch::Entry* e, const char* context, const void* const* inputs, const size_t* lens,
                      size_t n_inputs, size_t expected_bytes, void* dst) {
    if (e->inputs.size() != n_inputs)
        return bad_inputs("Fix: " + std::string(context) + " passes " + std::to_string(n_inputs) +
                          " input buffer(s) but the Program declares " + std::to_string(e->inputs.size()) + ".");
    std::vector<vyb_binding> b(n_inputs);
    for (size_t i = 0; i < n_inputs; ++i) {
        b[i] = vyb_binding();
        b[i].value_id = e->inputs[i].binding;
        b[i].kind = VYB_BIND_HOST;
        b[i].host_ptr = inputs[i];
        b[i].len = lens[i];
    }
    vyb_submission* sub = nullptr;
    vyb_completion* done = nullptr;
    if (vyb_submit(e->instance, e->digest, b.data(), b.size(), nullptr, &sub) != VYB_OK ||
        vyb_submission_wait(sub, &done) != VYB_OK)
        return backend_error(vyb_last_error_message());
    int32_t rc = VYB_OK;
    if (e->outputs != 1 || vyb_completion_output_count(done) != 1) {
        rc = backend_error("Fix: " + std::string(context) + " expected exactly one output buffer, got " +
                           std::to_string(vyb_completion_output_count(done)) + ".");
    } else {
        const uint8_t* bytes = nullptr;
        size_t len = 0;
        if (vyb_completion_output(done, e->output_id, &bytes, &len) != VYB_OK) {
            rc = backend_error(vyb_last_error_message());
        } else if (len != expected_bytes) {
            rc = backend_error("Fix: " + std::string(context) + " expected " + std::to_string(expected_bytes) +
                               " output bytes, got " + std::to_string(len) + ".");
        } else {
            std::memcpy(dst, bytes, len);
        }
    }
    vyb_completion_free(done);
    return rc;
}

std::string dims3(uint32_t batch, uint32_t rows, uint32_t cols) {
    return "batch=" + std::to_string(batch) + " rows=" + std::to_string(rows) + " cols=" + std::to_string(cols);
}

// shapes.rs:12-76
int32_t validate_batched_packed_matmul_shape(const std::string& context, size_t weights_len, size_t activations_len,
                                             size_t row_scales_len, size_t batch_scales_len, uint32_t batch, uint32_t rows,
                                             uint32_t cols) {
    if (batch == 0 || rows == 0 || cols == 0)
        return bad_inputs("Fix: " + context + " requires batch > 0, rows > 0, and cols > 0, got " + dims3(batch, rows, cols) + ".");
    const size_t wpr = vyb_i4_packed_words(cols);
    const size_t expected_w = size_t(rows) * wpr, expected_a = size_t(batch) * wpr;
    if (weights_len != expected_w)
        return bad_inputs("Fix: " + context + " requires weights_packed.len() == rows*i4_packed_words(cols), got len=" +
                          std::to_string(weights_len) + " expected=" + std::to_string(expected_w) + " for rows=" +
                          std::to_string(rows) + " cols=" + std::to_string(cols) + ".");
    if (activations_len != expected_a)
        return bad_inputs("Fix: " + context + " requires activation_batches_packed.len() == batch*i4_packed_words(cols), got len=" +
                          std::to_string(activations_len) + " expected=" + std::to_string(expected_a) + " for batch=" +
                          std::to_string(batch) + " cols=" + std::to_string(cols) + ".");
    if (row_scales_len != rows)
        return bad_inputs("Fix: " + context + " requires row_scales.len() == rows, got len=" + std::to_string(row_scales_len) +
                          " rows=" + std::to_string(rows) + ".");
    if (batch_scales_len != batch)
        return bad_inputs("Fix: " + context + " requires batch_scales.len() == batch, got len=" +
                          std::to_string(batch_scales_len) + " batch=" + std::to_string(batch) + ".");
    if (uint64_t(batch) * rows > 0xFFFFFFFFull)
        return bad_inputs("Fix: " + context + " output grid overflows u32 for batch=" + std::to_string(batch) + " rows=" +
                          std::to_string(rows) + ".");
    return VYB_OK;
}

int32_t need(vyb_quantized_scratch* s, const void* out) {
    if (!s) return fail_invalid_program("Fix: pass a scratch made by vyb_quantized_scratch_new.");
    if (!out) return fail_invalid_program("Fix: pass a non-null output pointer.");
    return VYB_OK;
}

}  // namespace

extern "C" {

int32_t vyb_quantized_scratch_new(vyb_device* device, vyb_quantized_scratch** scratch) {
    // a scratch without a device still validates shapes (the reference's wrappers are tested against a dispatcher that is
    // never reached); every dispatch on it is Rejected
    if (!scratch) return fail_invalid_program("Fix: pass an output pointer.");
    *scratch = new vyb_quantized_scratch();
    (*scratch)->device = device;
    if (device) vyb_device_retain(device);  // the scratch materialises on this device until it is freed
    return VYB_OK;
}

void vyb_quantized_scratch_free(vyb_quantized_scratch* s) {
    if (!s) return;
    for (auto& kv : s->cache) drop(kv.second);
    if (s->device) vyb_device_release(s->device);
    delete s;
}

void vyb_quantized_scratch_stats(const vyb_quantized_scratch* s, uint64_t* cached, uint64_t* hits, uint64_t* misses) {
    if (cached) *cached = s ? s->cache.size() : 0;
    if (hits) *hits = s ? s->hits : 0;
    if (misses) *misses = s ? s->misses : 0;
}

int32_t vyb_unpack_i4x8_via(vyb_quantized_scratch* s, const uint32_t* packed_words, size_t packed_len, uint32_t lane_count,
                            int32_t* out_lanes) {
    if (int32_t rc = need(s, out_lanes)) return rc;
    if (lane_count == 0) return bad_inputs("Fix: unpack_i4x8_via requires lane_count > 0.");
    const size_t expected_words = vyb_i4_packed_words(lane_count);
    if (packed_len != expected_words)
        return bad_inputs("Fix: unpack_i4x8_via requires packed_words.len() == i4_packed_words(lane_count), got len=" +
                          std::to_string(packed_len) + " expected=" + std::to_string(expected_words) + " for lane_count=" +
                          std::to_string(lane_count) + ".");
    std::lock_guard<std::mutex> lock(s->mu);
    vyb_quantized_scratch::Entry* e = nullptr;
    if (int32_t rc = entry_for(s, {W_UNPACK, lane_count, 0, 0},
                               [&](vyb_program** p) { return vyb_math_unpack_i4x8("packed", "lanes", lane_count, p); }, &e))
        return rc;
    const size_t out_bytes = size_t(lane_count) * 4;
    if (e->inputs.size() == 2) {  // `lanes` declared ReadWrite: bound as zero bytes, like the reference
        if (s->zeros.size() < out_bytes) s->zeros.assign(out_bytes, 0);
        const void* in[2] = {packed_words, s->zeros.data()};
        const size_t len[2] = {packed_len * 4, out_bytes};
        return dispatch_into(e, "unpack_i4x8_via", in, len, 2, out_bytes, out_lanes);
    }
    const void* in[1] = {packed_words};
    const size_t len[1] = {packed_len * 4};
    return dispatch_into(e, "unpack_i4x8_via", in, len, 1, out_bytes, out_lanes);
}

int32_t vyb_i4x8_dot_f32_scaled_via(vyb_quantized_scratch* s, const uint32_t* lhs_packed, size_t lhs_len,
                                    const uint32_t* rhs_packed, size_t rhs_len, float lhs_scale, float rhs_scale,
                                    uint32_t lane_count, float* out) {
    if (int32_t rc = need(s, out)) return rc;
    if (lane_count == 0) return bad_inputs("Fix: i4x8_dot_f32_scaled_via requires lane_count > 0.");
    const size_t expected_words = vyb_i4_packed_words(lane_count);
    if (lhs_len != expected_words || rhs_len != expected_words)
        return bad_inputs("Fix: i4x8_dot_f32_scaled_via requires lhs/rhs packed lengths == i4_packed_words(lane_count), got lhs=" +
                          std::to_string(lhs_len) + " rhs=" + std::to_string(rhs_len) + " expected=" +
                          std::to_string(expected_words) + " for lane_count=" + std::to_string(lane_count) + ".");
    std::lock_guard<std::mutex> lock(s->mu);
    vyb_quantized_scratch::Entry* e = nullptr;
    if (int32_t rc = entry_for(s, {W_DOT, lane_count, 0, 0}, [&](vyb_program** p) {
            return vyb_math_i4x8_dot_f32_scaled("lhs", "rhs", "lhs_scale", "rhs_scale", "out", lane_count, 0, p);
        }, &e))
        return rc;
    const void* in[4] = {lhs_packed, rhs_packed, &lhs_scale, &rhs_scale};
    const size_t len[4] = {lhs_len * 4, rhs_len * 4, 4, 4};
    return dispatch_into(e, "i4x8_dot_f32_scaled_via", in, len, 4, 4, out);
}

int32_t vyb_i4x8_matvec_f32_scaled_via(vyb_quantized_scratch* s, const uint32_t* weights_packed, size_t weights_len,
                                       const float* x, size_t x_len, const float* row_scales, size_t row_scales_len,
                                       uint32_t rows, uint32_t cols, float* out) {
    if (int32_t rc = need(s, out)) return rc;
    const std::string ctx = "i4x8_matvec_f32_scaled_via";
    if (rows == 0 || cols == 0)
        return bad_inputs("Fix: " + ctx + " requires rows > 0 and cols > 0, got rows=" + std::to_string(rows) + " cols=" +
                          std::to_string(cols) + ".");
    const size_t expected_w = size_t(rows) * vyb_i4_packed_words(cols);
    if (weights_len != expected_w)
        return bad_inputs("Fix: " + ctx + " requires weights_packed.len() == rows*i4_packed_words(cols), got len=" +
                          std::to_string(weights_len) + " expected=" + std::to_string(expected_w) + " for rows=" +
                          std::to_string(rows) + " cols=" + std::to_string(cols) + ".");
    if (x_len != cols)
        return bad_inputs("Fix: " + ctx + " requires x.len() == cols, got len=" + std::to_string(x_len) + " cols=" +
                          std::to_string(cols) + ".");
    if (row_scales_len != rows)
        return bad_inputs("Fix: " + ctx + " requires row_scales.len() == rows, got len=" + std::to_string(row_scales_len) +
                          " rows=" + std::to_string(rows) + ".");
    std::lock_guard<std::mutex> lock(s->mu);
    vyb_quantized_scratch::Entry* e = nullptr;
    if (int32_t rc = entry_for(s, {W_MATVEC, rows, cols, 0}, [&](vyb_program** p) {
            return vyb_math_i4x8_matvec_f32_scaled("weights", "x", "row_scales", "out", rows, cols, 0, p);
        }, &e))
        return rc;
    const void* in[3] = {weights_packed, x, row_scales};
    const size_t len[3] = {weights_len * 4, x_len * 4, row_scales_len * 4};
    return dispatch_into(e, ctx.c_str(), in, len, 3, size_t(rows) * 4, out);
}

int32_t vyb_i4x8_batched_matvec_f32_scaled_via(vyb_quantized_scratch* s, const uint32_t* weights_packed, size_t weights_len,
                                               const float* x_batches, size_t x_len, const float* row_scales,
                                               size_t row_scales_len, uint32_t batch, uint32_t rows, uint32_t cols,
                                               float* out) {
    if (int32_t rc = need(s, out)) return rc;
    const std::string ctx = "i4x8_batched_matvec_f32_scaled_via";
    if (batch == 0 || rows == 0 || cols == 0)
        return bad_inputs("Fix: " + ctx + " requires batch > 0, rows > 0, and cols > 0, got " + dims3(batch, rows, cols) + ".");
    const size_t expected_w = size_t(rows) * vyb_i4_packed_words(cols);
    if (weights_len != expected_w)
        return bad_inputs("Fix: " + ctx + " requires weights_packed.len() == rows*i4_packed_words(cols), got len=" +
                          std::to_string(weights_len) + " expected=" + std::to_string(expected_w) + " for rows=" +
                          std::to_string(rows) + " cols=" + std::to_string(cols) + ".");
    const size_t expected_x = size_t(batch) * cols;
    if (x_len != expected_x)
        return bad_inputs("Fix: " + ctx + " requires x_batches.len() == batch*cols, got len=" + std::to_string(x_len) +
                          " expected=" + std::to_string(expected_x) + " for batch=" + std::to_string(batch) + " cols=" +
                          std::to_string(cols) + ".");
    if (row_scales_len != rows)
        return bad_inputs("Fix: " + ctx + " requires row_scales.len() == rows, got len=" + std::to_string(row_scales_len) +
                          " rows=" + std::to_string(rows) + ".");
    std::lock_guard<std::mutex> lock(s->mu);
    vyb_quantized_scratch::Entry* e = nullptr;
    if (int32_t rc = entry_for(s, {W_BATCHED_MATVEC, batch, rows, cols}, [&](vyb_program** p) {
            return vyb_math_i4x8_batched_matvec_f32_scaled("weights", "x_batches", "row_scales", "out", batch, rows, cols, 0, p);
        }, &e))
        return rc;
    const void* in[3] = {weights_packed, x_batches, row_scales};
    const size_t len[3] = {weights_len * 4, x_len * 4, row_scales_len * 4};
    return dispatch_into(e, ctx.c_str(), in, len, 3, size_t(batch) * rows * 4, out);
}

int32_t vyb_i4x8_batched_matmul_f32_scaled_via(vyb_quantized_scratch* s, const uint32_t* weights_packed, size_t weights_len,
                                               const uint32_t* activation_batches_packed, size_t activations_len,
                                               const float* row_scales, size_t row_scales_len, const float* batch_scales,
                                               size_t batch_scales_len, uint32_t batch, uint32_t rows, uint32_t cols,
                                               float* out) {
    if (int32_t rc = need(s, out)) return rc;
    const std::string ctx = "i4x8_batched_matmul_f32_scaled_via";
    if (int32_t rc = validate_batched_packed_matmul_shape(ctx, weights_len, activations_len, row_scales_len, batch_scales_len,
                                                          batch, rows, cols))
        return rc;
    std::lock_guard<std::mutex> lock(s->mu);
    vyb_quantized_scratch::Entry* e = nullptr;
    if (int32_t rc = entry_for(s, {W_BATCHED_MATMUL, batch, rows, cols}, [&](vyb_program** p) {
            return vyb_math_i4x8_batched_matmul_f32_scaled("weights", "activations", "row_scales", "batch_scales", "out", batch,
                                                           rows, cols, 0, p);
        }, &e))
        return rc;
    const void* in[4] = {weights_packed, activation_batches_packed, row_scales, batch_scales};
    const size_t len[4] = {weights_len * 4, activations_len * 4, row_scales_len * 4, batch_scales_len * 4};
    return dispatch_into(e, ctx.c_str(), in, len, 4, size_t(batch) * rows * 4, out);
}

int32_t vyb_i4x8_batched_matmul_top1_f32_scaled_via(vyb_quantized_scratch* s, const uint32_t* weights_packed,
                                                    size_t weights_len, const uint32_t* activation_batches_packed,
                                                    size_t activations_len, const float* row_scales, size_t row_scales_len,
                                                    const float* batch_scales, size_t batch_scales_len, uint32_t batch,
                                                    uint32_t rows, uint32_t cols, float* scores_out, uint32_t* indices_out) {
    if (int32_t rc = need(s, scores_out)) return rc;
    if (!indices_out) return fail_invalid_program("Fix: pass a non-null output pointer.");
    const std::string ctx = "i4x8_batched_matmul_top1_f32_scaled_via";
    if (int32_t rc = validate_batched_packed_matmul_shape(ctx, weights_len, activations_len, row_scales_len, batch_scales_len,
                                                          batch, rows, cols))
        return rc;
    std::lock_guard<std::mutex> lock(s->mu);
    vyb_quantized_scratch::Entry* e = nullptr;
    if (int32_t rc = entry_for(s, {W_TOP1, batch, rows, cols}, [&](vyb_program** p) {
            return vyb_math_i4x8_batched_matmul_top1_f32_scaled("weights", "activations", "row_scales", "batch_scales", "scores",
                                                                batch, rows, cols, 0, p);
        }, &e))
        return rc;
    // one buffer of batch * 2 f32: the best scores, then the best indices cast to f32 (top1.rs:86-110)
    std::vector<float> both(size_t(batch) * 2);
    const void* in[4] = {weights_packed, activation_batches_packed, row_scales, batch_scales};
    const size_t len[4] = {weights_len * 4, activations_len * 4, row_scales_len * 4, batch_scales_len * 4};
    if (int32_t rc = dispatch_into(e, ctx.c_str(), in, len, 4, both.size() * 4, both.data())) return rc;
    for (uint32_t b = 0; b < batch; ++b) {
        scores_out[b] = both[b];
        indices_out[b] = uint32_t(both[size_t(batch) + b]);
    }
    return VYB_OK;
}

}  // extern "C"
