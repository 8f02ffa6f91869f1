"""The reference's authenticated frames (VMK0 / VTP0 / VME0) around this backend's target bytes: the framing rule is
restated in Python from vyre-megakernel/src/envelope.rs:763-786, 861-877 and lib.rs:1326-1355 and compared byte for byte;
the TargetPayloadBody is compared with the compact serde_json form of its fields in declaration order
(envelope.rs:182-192); the reference's decode checks (envelope.rs:788-860) are hit one by one. No vector of the reference
pins frame bytes (its tests build frames with the same rule at run time): parity unpinned, rule restated."""
import json
import struct

import pytest

import vyre_b200 as vb
from vyre_b200 import api, ffi

LAYERS = {api.FRAME_VMK0: (b"VMK0", 4, b"vyre-megakernel-artifact-v4\0"),
          api.FRAME_VTP0: (b"VTP0", 3, b"vyre-megakernel-target-payload-v3\0"),
          api.FRAME_VME0: (b"VME0", 2, b"vyre-megakernel-envelope-v2\0")}


def blake3(data: bytes) -> bytes:
    out = (ffi.C.c_char * 32)()
    ffi.lib().vyb_blake3(data, len(data), out)
    return out.raw


def frame_by_rule(layer: int, body: bytes) -> bytes:
    magic, schema, domain = LAYERS[layer]
    digest = blake3(domain + struct.pack("<H", schema) + struct.pack("<Q", len(body)) + body)
    return magic + struct.pack("<H", schema) + struct.pack("<I", len(body)) + body + digest


@pytest.mark.parametrize("layer", [0, 1, 2])
def test_framing_matches_the_rule_and_decodes(layer):
    for body in (b"", b"{}", b'{"schema_version":4,"nodes":[]}' * 50):
        frame = api.frame_encode(layer, body)
        assert frame == frame_by_rule(layer, body)
        got, digest = api.frame_decode(layer, frame)
        assert got == body and digest == frame[-32:]


def test_decode_checks_in_the_reference_order():
    frame = api.frame_encode(api.FRAME_VTP0, b'{"x":1}')
    def refused(data, text, layer=api.FRAME_VTP0):
        with pytest.raises(vb.BackendError) as e:
            api.frame_decode(layer, data)
        assert text in e.value.message and "Fix:" in e.value.message
    refused(frame[:20], "target_payload.header: framed bytes are shorter than the fixed header and digest")
    refused(frame, "envelope.magic: framing magic is invalid", layer=api.FRAME_VME0)
    refused(b"VTP0" + struct.pack("<H", 2) + frame[6:], "target_payload.schema_version: schema 2 is unsupported; expected 3")
    refused(frame + b"\0", f"target_payload.body_length: framing declares {len(frame)} bytes but received {len(frame) + 1}")
    tampered = bytearray(frame)
    tampered[12] ^= 1
    refused(bytes(tampered), "target_payload.digest: framed body does not match its content identity")


def a_payload():
    prog = vb.linear_4bit_affine_grouped("x", "w", "scale", "zp", "b", "out", 64, 16, 32)
    art = vb.compile(prog)
    return prog, art, vb.target_compile(art)


def test_target_payload_body_is_the_reference_struct_in_compact_json():
    prog, art, payload = a_payload()
    neutral = bytes(range(32))
    frame = api.payload_to_vtp0(payload, neutral, node_id=3)
    body, digest = api.frame_decode(api.FRAME_VTP0, frame)
    obj = json.loads(body)
    assert body == json.dumps(obj, separators=(",", ":")).encode()  # compact, as serde_json::to_vec writes it
    assert list(obj) == ["schema_version", "neutral_artifact", "format", "profile", "entries", "bytes"]
    assert obj["schema_version"] == 3 and obj["neutral_artifact"] == list(neutral)
    assert obj["format"] == {"identity": payload.format(), "version": 1}
    assert list(obj["profile"]) == ["identity", "generation", "max_workgroup_size", "max_invocations_per_workgroup",
                                    "max_dynamic_shared_bytes", "subgroup_size"]
    assert obj["profile"]["generation"] > 0 and obj["profile"]["subgroup_size"] == 32
    (entry,) = obj["entries"]
    assert list(entry) == ["name", "node", "workgroup_size", "grid_size", "dynamic_shared_bytes", "resource_bindings"]
    assert entry["name"] == "main" and entry["node"] == 3 and entry["workgroup_size"] == list(prog.workgroup_size())
    slots = [b["binding"] for b in prog.buffers() if b["access"] != ffi.ACCESS_WORKGROUP]
    assert [r["slot"] for r in entry["resource_bindings"]] == sorted(slots)
    assert all(list(r) == ["resource", "group", "slot", "memory", "access"] and r["memory"] == "global" for r in entry["resource_bindings"])
    assert {r["access"] for r in entry["resource_bindings"]} == {"read_only", "write_only"}
    assert bytes(obj["bytes"]) == payload.to_bytes()
    # caller-supplied ArtifactValueIds
    ids = [100 + i for i in range(len(slots))]
    obj2 = json.loads(api.frame_decode(api.FRAME_VTP0, api.payload_to_vtp0(payload, neutral, 0, ids))[0])
    assert [r["resource"] for r in obj2["entries"][0]["resource_bindings"]] == ids
    with pytest.raises(vb.BackendError, match="one ArtifactValueId per bound buffer"):
        api.payload_to_vtp0(payload, neutral, 0, [1, 2])
    # and back: the same target bytes, the same payload identity, the digest it was bound to
    again, bound = api.payload_from_vtp0(frame)
    assert again.to_bytes() == payload.to_bytes() and again.digest() == payload.digest() and bound == neutral


def test_payload_from_vtp0_refuses_foreign_or_inconsistent_bodies():
    _, _, payload = a_payload()
    body = json.loads(api.frame_decode(api.FRAME_VTP0, api.payload_to_vtp0(payload, bytes(32)))[0])
    def reframed(obj):
        return api.frame_encode(api.FRAME_VTP0, json.dumps(obj, separators=(",", ":")).encode())
    with pytest.raises(vb.BackendError, match="format identity or version differs"):
        api.payload_from_vtp0(reframed({**body, "format": {"identity": "someone-else", "version": 1}}))
    with pytest.raises(vb.BackendError, match="neutral_artifact is not a 32-byte digest"):
        api.payload_from_vtp0(reframed({**body, "neutral_artifact": [1, 2, 3]}))
    with pytest.raises(vb.BackendError):
        api.payload_from_vtp0(reframed({**body, "bytes": body["bytes"][:-1]}))  # the target bytes authenticate themselves
    with pytest.raises(vb.BackendError, match="not a TargetPayloadBody"):
        api.payload_from_vtp0(api.frame_encode(api.FRAME_VTP0, b'{"neutral_artifact":[]}'))


def test_envelope_carries_the_neutral_frame_and_bound_payloads():
    _, _, payload = a_payload()
    vmk0 = api.frame_encode(api.FRAME_VMK0, b'{"schema_version":4,"nodes":[],"dependencies":[]}')  # stands in for vyre's artifact
    neutral = vmk0[-32:]  # Artifact::digest() is the frame's digest (lib.rs:1345-1352)
    vtp0 = api.payload_to_vtp0(payload, neutral)
    vme0 = api.envelope_to_vme0(vmk0, [vtp0, vtp0])
    body = json.loads(api.frame_decode(api.FRAME_VME0, vme0)[0])
    assert list(body) == ["schema_version", "neutral_artifact", "target_payloads"] and body["schema_version"] == 2
    assert bytes(body["neutral_artifact"]) == vmk0 and [bytes(p) for p in body["target_payloads"]] == [vtp0, vtp0]
    assert api.envelope_from_vme0(vme0) == (vmk0, [vtp0, vtp0])
    assert api.envelope_from_vme0(api.envelope_to_vme0(vmk0, [])) == (vmk0, [])
    other = api.payload_to_vtp0(payload, bytes(32))
    with pytest.raises(vb.BackendError, match="bound to another neutral artifact"):
        api.envelope_to_vme0(vmk0, [other])
    with pytest.raises(vb.BackendError, match="artifact.magic"):
        api.envelope_to_vme0(vtp0, [])
