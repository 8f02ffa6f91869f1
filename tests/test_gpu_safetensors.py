"""Weights from a safetensors shard to resident device buffers to a submission: the tensor bytes go file -> device
(vyb_safetensors_upload), bind as resident values, and the decode GEMV through the contract path gives the same bytes
as with weights uploaded from host arrays."""
import json
import struct

import numpy as np
import pytest

import vyre_b200 as vb
from vyre_b200 import api, ffi, synth

pytestmark = pytest.mark.gpu


def test_int4_linear_with_weights_loaded_from_a_safetensors_shard(tmp_path):
    m, n, k = 2, 640, 4096
    x, w, s = synth.int4_linear_inputs(m, n, k, seed=21)
    wb, sb = w.tobytes(), s.tobytes()
    pad = b"\0" * 24  # tensors need not be adjacent
    header = {"layers.0.mlp.w.qweight": {"dtype": "U8", "shape": [n, k // 2], "data_offsets": [0, len(wb)]},
              "layers.0.mlp.w.scales": {"dtype": "BF16", "shape": [n, k // 128], "data_offsets": [len(wb) + 24, len(wb) + 24 + len(sb)]},
              "__metadata__": {"quant": "int4-g128"}}
    raw = json.dumps(header).encode()
    path = tmp_path / "shard.safetensors"
    path.write_bytes(struct.pack("<Q", len(raw)) + raw + wb + pad + sb)

    dev = vb.Device.acquire(0)
    try:
        idx = api.SafetensorIndex.open(str(path))
        idx.require("layers.0.mlp.w.qweight", "U8", [n, k // 2])
        idx.require("layers.0.mlp.w.scales", "BF16", [n, k // 128])
        hw = idx.load_resident(dev, "layers.0.mlp.w.qweight")
        hs = idx.load_resident(dev, "layers.0.mlp.w.scales")
        assert dev.download_resident(hw, len(wb)).tobytes() == wb and dev.download_resident(hs, len(sb)).tobytes() == sb
        # into the middle of a larger buffer, too
        big = dev.allocate_resident(len(sb) + 512)
        idx.load_resident(dev, "layers.0.mlp.w.scales", handle=big, offset=256)
        assert dev.download_resident(big, len(sb), offset=256).tobytes() == sb

        sess = vb.ArtifactSession.compile(vb.linear_int4_grouped_rowmajor("x", "w", "scale", "out", m, k, n, 128, ffi.DT_BF16), dev)

        def run(hw_, hs_):
            bs = vb.BindingSet(sess.artifact.digest())
            bs.insert_host(0, x)
            bs.insert_resident(1, hw_)
            bs.insert_resident(2, hs_)
            return sess.submit(bs).wait().output(3)

        from_file = run(hw, hs)
        from_host = run(dev.resident_from(w.view(np.uint32)), dev.resident_from(s))
        assert from_file == from_host and len(from_file) == m * n * 2
        # a shard that changed after it was indexed is refused before any byte moves
        path.write_bytes(path.read_bytes() + b"\0")
        with pytest.raises(vb.BackendError, match="changed length"):
            idx.load_resident(dev, "layers.0.mlp.w.scales")
    finally:
        dev.release()
