"""CPU-only checks of the host side: the C-ABI library loads and exports every declared symbol, the operator
builders keep the reference's validation texts and storage known-answers, artifacts/payloads authenticate, and
a missing device is a structured failure. No compute is launched here."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import vyre_b200 as vb
from vyre_b200 import ffi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "vyre_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vyb_[a-z0-9_]+)\s*\(", text)))


def test_library_loads_and_exports_every_declared_symbol():
    L = ffi.lib()
    names = declared_symbols()
    assert len(names) > 70
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/vyre_b200.h but not exported"
    assert set(ffi.exported_names()) == set(names), set(ffi.exported_names()) ^ set(names)
    assert L.vyb_abi_version() == 1


# ---- blake3 (digest of Artifact / TargetPayload identities) --------------------------------------------------
def _blake3_py(data: bytes) -> bytes:
    """Independent recursive formulation of BLAKE3 used only to cross-check the library's incremental one."""
    IV = [0x6A09E667, 0xBB67AE85, 0x3C6EF372, 0xA54FF53A, 0x510E527F, 0x9B05688C, 0x1F83D9AB, 0x5BE0CD19]
    PERM = [2, 6, 3, 10, 7, 0, 4, 13, 1, 11, 12, 5, 9, 14, 15, 8]
    M = 0xFFFFFFFF

    def rotr(x, n):
        return ((x >> n) | (x << (32 - n))) & M

    def g(s, a, b, c, d, mx, my):
        s[a] = (s[a] + s[b] + mx) & M
        s[d] = rotr(s[d] ^ s[a], 16)
        s[c] = (s[c] + s[d]) & M
        s[b] = rotr(s[b] ^ s[c], 12)
        s[a] = (s[a] + s[b] + my) & M
        s[d] = rotr(s[d] ^ s[a], 8)
        s[c] = (s[c] + s[d]) & M
        s[b] = rotr(s[b] ^ s[c], 7)

    def compress(cv, m, counter, blen, flags):
        s = cv[:] + IV[:4] + [counter & M, (counter >> 32) & M, blen, flags]
        m = m[:]
        for r in range(7):
            g(s, 0, 4, 8, 12, m[0], m[1]); g(s, 1, 5, 9, 13, m[2], m[3])
            g(s, 2, 6, 10, 14, m[4], m[5]); g(s, 3, 7, 11, 15, m[6], m[7])
            g(s, 0, 5, 10, 15, m[8], m[9]); g(s, 1, 6, 11, 12, m[10], m[11])
            g(s, 2, 7, 8, 13, m[12], m[13]); g(s, 3, 4, 9, 14, m[14], m[15])
            m = [m[PERM[i]] for i in range(16)]
        return [s[i] ^ s[i + 8] for i in range(8)]

    def words(b):
        b = b + bytes(64 - len(b))
        return [int.from_bytes(b[4 * i:4 * i + 4], "little") for i in range(16)]

    def chunk_cv(chunk, counter, root):
        cv = IV[:]
        blocks = [chunk[i:i + 64] for i in range(0, len(chunk), 64)] or [b""]
        for i, blk in enumerate(blocks):
            flags = (1 if i == 0 else 0) | (2 if i == len(blocks) - 1 else 0)
            if root and i == len(blocks) - 1:
                flags |= 8
            cv = compress(cv, words(blk), counter, len(blk), flags)
        return cv

    def subtree(data, counter0, root):
        nchunks = max(1, (len(data) + 1023) // 1024)
        if nchunks == 1:
            return chunk_cv(data, counter0, root)
        left = 1 << ((nchunks - 1).bit_length() - 1)  # largest power of two strictly below nchunks
        l = subtree(data[:left * 1024], counter0, False)
        r = subtree(data[left * 1024:], counter0 + left, False)
        return compress(IV[:], l + r, 0, 64, 4 | (8 if root else 0))

    return b"".join(w.to_bytes(4, "little") for w in subtree(data, 0, True))


def test_blake3_known_answers_and_tree_structure():
    assert vb.blake3(b"").hex() == "af1349b9f5f9a1a6a0404dea36dcc9499bcb25c9adc112b7cc9a93cae41f3262"
    assert vb.blake3(b"abc").hex() == "6437b3ac38465133ffb63b75273a8db548c558465d79db03fd359c6cd5bd9d85"
    pattern = bytes(i % 251 for i in range(8192))
    for n in [0, 1, 63, 64, 65, 1023, 1024, 1025, 2048, 2049, 3072, 3073, 4096, 5000, 7169, 8192]:
        assert vb.blake3(pattern[:n]) == _blake3_py(pattern[:n]), n


# ---- builders: validation texts (linear_4bit.rs:263-277, 411-455) -------------------------------------------------
def test_linear_4bit_builder_rejections():
    with pytest.raises(vb.BackendError, match="divisible by 8") as e:
        vb.linear_4bit("x", "w", "b", "out", 7, 4)
    assert e.value.code == ffi.ERR_INVALID_PROGRAM and e.value.message.startswith("Fix:")
    with pytest.raises(vb.BackendError, match="in_dim=0"):
        vb.linear_4bit("x", "w", "b", "out", 0, 4)
    with pytest.raises(vb.BackendError, match="out_dim=0"):
        vb.linear_4bit("x", "w", "b", "out", 8, 0)
    with pytest.raises(vb.BackendError, match="overflows u32"):
        vb.linear_4bit("x", "w", "b", "out", 0xFFFFFFF8, 16)


def test_affine_grouped_builder_rejections_and_padding():
    for kw, pat in [((0, 2, 4, 1), "in_dim=0"), ((8, 0, 4, 1), "out_dim=0"), ((8, 2, 0, 1), "group_size=0"),
                    ((8, 2, 4, 0), "batch_size=0"), ((12, 2, 4, 1), "divisible by 8")]:
        with pytest.raises(vb.BackendError, match=pat):
            vb.linear_4bit_affine_grouped_batched("x", "w", "s", "zp", "b", "out", *kw)
    p = vb.linear_4bit_affine_grouped("x", "w", "scale", "zp", "b", "out", 8, 2, 4)
    assert p.op_id == "vyre-libs::nn::linear_4bit_affine_grouped"
    assert p.workgroup_size() == [256, 1, 1]
    bufs = p.buffers()
    assert [b["binding"] for b in bufs] == [0, 1, 2, 3, 4, 5]
    assert [b["count"] for b in bufs[:5]] == [8, 2, 4, 4, 2]
    # output padded to ceil(B*N/8)*256 elements, trimmed by output_byte_range (linear_4bit.rs:743-771)
    assert bufs[5]["count"] == 256 and bufs[5]["output_byte_range"] == (0, 8)
    # generated sweep of the reference (linear_4bit.rs:1570-1608)
    accepted = rejected = 0
    for in_dim in [8, 10, 16, 18, 24, 32, 64, 128]:
        for out_dim in [1, 2, 3, 7, 16, 31]:
            for g in [1, 2, 4, 8, 16, 32]:
                spec = vb.QuantizedLinear4BitSpec.affine_grouped(in_dim, out_dim, g)
                if in_dim % 8 == 0:
                    out = vb.linear_4bit_affine_grouped_typed(spec, "x", "w", "scale", "zp", "b", "out").buffers()[5]
                    assert out["count"] >= out_dim and out["output_byte_range"] == (0, out_dim * 4)
                    accepted += 1
                else:
                    with pytest.raises(vb.BackendError, match="divisible by 8"):
                        vb.linear_4bit_affine_grouped_typed(spec, "x", "w", "scale", "zp", "b", "out")
                    rejected += 1
    assert accepted + rejected >= 216
    # weight-reuse variant declares the workgroup tile and (batch/8)*out_dim workgroups (linear_4bit.rs:778-811)
    p = vb.linear_4bit_affine_grouped_batched("x", "w", "scale", "zp", "b", "out", 256, 8, 64, 8)
    names = [b["name"] for b in p.buffers()]
    assert "linear_4bit_weight_tile" in names
    assert [b for b in p.buffers() if b["name"] == "out"][0]["count"] == 8 * 256
    p = vb.linear_4bit_affine_grouped_batched("linear_4bit_weight_tile", "w", "scale", "zp", "b", "out", 256, 8, 64, 8)
    assert sum(b["name"] == "linear_4bit_weight_tile" for b in p.buffers()) == 1


def test_typed_spec_metadata_contract():
    bad_storage = vb.QuantizedLinear4BitSpec(32, 4, ffi.DT_I8, 8, 8)
    with pytest.raises(vb.BackendError, match="storage I4"):
        vb.linear_4bit_affine_grouped_typed(bad_storage, "x", "w", "scale", "zp", "b", "out")
    bad_sidecar = vb.QuantizedLinear4BitSpec(32, 4, ffi.DT_I4, 8, 16)
    with pytest.raises(vb.BackendError, match="group sizes to match"):
        vb.linear_4bit_affine_grouped_typed(bad_sidecar, "x", "w", "scale", "zp", "b", "out")


def test_planner_evidence_known_answer():
    # linear_4bit.rs:1497-1530
    ev = vb.linear_4bit_affine_grouped_planner_evidence(vb.QuantizedLinear4BitSpec.affine_grouped(256, 4096, 64))
    assert ev["group_count"] == 4
    assert ev["packed_weight_bytes"] == 524_288
    assert ev["dequantized_weight_bytes"] == 4_194_304 == ev["dequant_bytes_elided"]
    assert ev["sidecar_bytes"] == 131_072
    assert ev["bias_bytes"] == 16_384 and ev["output_bytes"] == 16_384
    assert (ev["matmul_m"], ev["matmul_k"], ev["matmul_n"], ev["matmul_tile"]) == (4096, 256, 1, 32)
    assert ev["matmul_selected_path"] == "cooperative" and ev["matmul_candidate_path"] is None
    assert ev["matmul_fallback_reason"] == "strict_f32_requested" and not ev["tensor_core_eligible"]
    assert np.float32(ev["output_drift_abs_tolerance"]) == np.float32(1e-4)


def test_int4_primitive_layout_known_answers_and_traps():
    # vyre-primitives/src/math/quantized/tests/layout_contracts.rs:1-108
    assert ffi.lib().vyb_i4_packed_words(65) == 9
    p = vb.i4x8_matvec_f32_scaled("w", "x", "s", "out", 3, 65)
    assert [b["count"] for b in p.buffers()] == [27, 65, 3, 3]
    assert p.op_id == "vyre-primitives::math::quantized::i4x8_matvec_f32_scaled"
    p = vb.i4x8_batched_matvec_f32_scaled("w", "x", "s", "out", 4, 3, 65)
    assert [b["count"] for b in p.buffers()] == [27, 260, 3, 12]
    p = vb.i4x8_batched_matmul_top1_f32_scaled("w", "a", "rs", "bs", "out", 4, 3, 65, lib_op_id=True)
    assert p.buffers()[4]["count"] == 8 and p.op_id == "vyre-libs::quant::int4_batched_matmul_top1_f32_scaled"
    # zero shapes become trap programs, never host errors (zero_shape_contracts.rs), and do not compile
    for prog in [vb.unpack_i4x8("p", "o", 0), vb.i4x8_dot_i32("l", "r", "o", 0),
                 vb.i4x8_matvec_f32_scaled("w", "x", "s", "o", 0, 8),
                 vb.i4x8_batched_matmul_f32_scaled("w", "a", "rs", "bs", "o", 1, 0, 8), vb.softmax_top_k("s", "i", "w", 8, 0),
                 vb.top_k("s", "i", 8, 0), vb.swiglu("g", "u", "o", 0)]:
        assert prog.is_trap and prog.trap_message.startswith("Fix:")
        assert len(prog.buffers()) == 1 and prog.buffers()[0]["count"] == 1
        with pytest.raises(vb.BackendError) as e:
            vb.compile(prog)
        assert e.value.code == ffi.ERR_INVALID_PROGRAM


def test_moe_and_linear_rows_builder_contracts():
    g = vb.moe_gate("scores", "indices", "weights", 8, 2)
    b = g.buffers()
    assert [(x["name"], x["binding"], x["access"]) for x in b[:3]] == [
        ("scores", 0, ffi.ACCESS_READ_ONLY), ("indices", 1, ffi.ACCESS_READ_WRITE), ("weights", 2, ffi.ACCESS_OUTPUT)]
    assert sum(x["access"] == ffi.ACCESS_OUTPUT for x in b) == 1  # V022: one ::output buffer
    s = vb.softmax_top_k("scores", "oi", "ow", 8, 2).buffers()
    assert [x["name"] for x in s] == ["scores", "oi", "ow", "best_vals", "best_idxs"]
    with pytest.raises(vb.BackendError, match="all dims must be > 0"):
        vb.expert_mlp("x", "wg", "bg", "wu", "bu", "wd", "bd", "out", 0, 2, 2)
    with pytest.raises(vb.BackendError, match="k cannot exceed num_experts"):
        vb.moe_layer_route_and_accumulate("x", "wr", "br", "ei", "ew", "eo", "out", 2, 2, 2, 3)
    with pytest.raises(vb.BackendError, match="nonzero rows"):
        vb.linear_rows("x", "w", "b", "out", 0, 2, 2)
    with pytest.raises(vb.BackendError, match="F16, BF16, or F32"):
        vb.linear_rows_no_bias_typed("x", "w", "out", 1, 2, 2, ffi.DT_U32)
    with pytest.raises(vb.BackendError, match="swiglu_typed requires n > 0"):
        vb.swiglu_typed("g", "u", "o", 0, ffi.DT_BF16)
    lr = vb.linear_rows("x", "w", "b", "out", 2, 3, 4).buffers()
    assert [x["binding"] for x in lr] == [0, 1, 2, 3] and lr[3]["count"] == 8
    assert vb.linear_rows_no_bias("x", "w", "out", 2, 3, 4).buffers()[2]["binding"] == 2


def test_registration_and_supported_ops():
    r = vb.registration()
    assert r["id"] == "cuda-b200" and r["payload_format"] == "b200-native" and r["format_version"] == 1
    assert r["profile"]["generation"] == 100 and r["profile"]["subgroup_size"] == 32
    assert r["profile"]["max_dynamic_shared_bytes"] == 232448
    ops = vb.supported_ops()
    for op in ["vyre-libs::nn::linear_4bit", "vyre-libs::nn::linear_4bit_affine_grouped", "vyre-libs::nn::linear_rows",
               "vyre-libs::quant::int4_dot_i32", "vyre-primitives::math::quantized::unpack_i4x8",
               "vyre-libs::quant::int8_unpack", "vyre-libs::nn::moe_gate", "vyre-libs::nn::softmax_top_k",
               "vyre-libs::nn::top_k", "vyre-libs::nn::moe::expert_mlp", "vyre-libs::nn::moe_layer_accumulate",
               "vyre-libs::nn::swiglu"]:
        assert op in ops


# ---- artifact / payload identity -------------------------------------------------------------------------------------
def test_artifact_and_payload_are_digest_bound_and_authenticated():
    p1 = vb.linear_4bit("x", "w", "b", "out", 8, 4)
    p2 = vb.linear_4bit("x", "w", "b", "out", 8, 4)
    p3 = vb.linear_4bit("x", "w", "b", "out", 16, 4)
    assert p1.fingerprint() == p2.fingerprint() != p3.fingerprint()
    a1, a3 = vb.compile(p1), vb.compile(p3)
    assert a1.digest() == vb.compile(p2).digest() != a3.digest()
    t1 = vb.target_compile(a1)
    assert t1.neutral_artifact() == a1.digest() and t1.format() == "b200-native"
    raw = t1.to_bytes()
    again = vb.TargetPayload.from_bytes(raw)
    assert again.digest() == t1.digest() and again.to_bytes() == raw
    tampered = bytearray(raw)
    tampered[40] ^= 1
    with pytest.raises(vb.BackendError, match="digest does not match") as e:
        vb.TargetPayload.from_bytes(bytes(tampered))
    assert e.value.code == ffi.ERR_INVALID_PROGRAM
    with pytest.raises(vb.BackendError):
        vb.TargetPayload.from_bytes(raw[:-5])


def test_binding_set_rejects_zero_grid_axis():
    bs = vb.BindingSet(b"\0" * 32)
    with pytest.raises(vb.BackendError, match="axis 1 must be positive"):
        bs.set_invocation_grid([4, 0, 1])


@pytest.mark.skipif(os.path.exists("/dev/nvidiactl"), reason="a device is present on this box")
def test_missing_device_is_a_structured_failure_not_a_fallback():
    with pytest.raises(vb.BackendError) as e:
        vb.Device.acquire(0)
    assert e.value.code == ffi.ERR_DISPATCH_FAILED
    assert "Fix:" in e.value.message and "no CPU path" in e.value.message
    # the kernel-level entry point refuses as well
    rc = ffi.lib().vyb_k_int4_gemv(C.c_void_p(16), C.c_void_p(16), C.c_void_p(16), C.c_void_p(16), 1, 16, 1024, 128,
                                   ffi.DT_BF16, None, None)
    assert rc == ffi.ERR_DISPATCH_FAILED
    assert b"Fix:" in ffi.lib().vyb_last_error_message()


def test_multi_gpu_contexts_are_validated_on_the_host():
    """Argument checks of the peer-memory entry points run before any device work: wrong worlds, missing peer
    addresses and unsupported sizes are structured errors with Fix: text."""
    import ctypes as C

    from vyre_b200 import ffi

    L = ffi.lib()
    ctx = ffi.AllGatherCtx()
    ctx.world, ctx.rank = 0, 0
    assert L.vyb_k_allgather_wait(C.byref(ctx), None, None) == ffi.ERR_INVALID_PROGRAM
    assert "Fix:" in L.vyb_last_error_message().decode()
    ctx.world, ctx.rank = 2, 2
    assert L.vyb_k_allgather_push(C.byref(ctx), 0, 1, 8, None, None) == ffi.ERR_INVALID_PROGRAM
    ctx.world, ctx.rank, ctx.epoch = 2, 0, 4096
    ctx.peer_out[0], ctx.peer_flag[0] = 4096, 8192          # rank 1's addresses are missing
    assert L.vyb_k_allgather_push(C.byref(ctx), 0, 1, 8, None, None) == ffi.ERR_INVALID_PROGRAM
    assert "every rank" in L.vyb_last_error_message().decode()

    ep = ffi.MoeEpCtx()
    sym, loc = C.c_uint64(0), C.c_uint64(0)
    assert L.vyb_k_moe_ep_sizes(512, 4096, 4096, 14336, 8, 2, 3, C.byref(ep), C.byref(sym), C.byref(loc)) == ffi.ERR_INVALID_PROGRAM
    assert L.vyb_k_moe_ep_sizes(512, 4096, 4096, 14336, 8, 2, 8, C.byref(ep), C.byref(sym), C.byref(loc)) == 0
    # worst case: all 8192 pairs of the job on one rank -> 8192 + 256 rows of 8 KB in, 1024 pairs of 8 KB back
    assert sym.value >= (8192 + 256) * 4096 * 2 + 512 * 2 * 4096 * 2 and ep.off_xg % 256 == 0 and ep.off_yhome > ep.off_xg
    assert loc.value >= (8192 + 256) * (14336 + 4096) * 2
    ep.world, ep.rank = 9, 0
    assert L.vyb_k_moe_ep_ffn_int4(C.byref(ep), 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 16, 16, 256, 256, 8, 2, 128, None, None) == ffi.ERR_INVALID_PROGRAM
