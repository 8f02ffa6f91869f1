"""Submission semantics of the contract path on a live device: host bytes are copied in at submit, every submission
reports its own kernel status, prepared (graph-replayed) submissions equal ordinary ones, and resident buffers bound
to work in flight are protected. Failures are injected on the host; no device fault is provoked.
"""
import numpy as np
import pytest

import oracle
import vyre_b200 as vb
from vyre_b200 import ffi, synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    d = vb.Device.acquire(0)
    yield d
    d.release()


def gemv_session(dev, m=1, n=512, k=4096):
    prog = vb.linear_int4_grouped_rowmajor("x", "w", "scale", "out", m, k, n, 128, ffi.DT_BF16)
    return vb.ArtifactSession.compile(prog, dev)


def test_host_bytes_are_copied_in_at_submit(dev):
    # BindingSet owns its host bytes (vyre-driver/src/backend/artifact_lifecycle.rs:34-96): a caller that rewrites its
    # buffer right after submit must still get the result of the bytes it submitted
    m, n, k = 1, 512, 4096
    x, w, s = synth.int4_linear_inputs(m, n, k, seed=11)
    sess = gemv_session(dev, m, n, k)
    want = sess.run_host([x, w.view(np.uint32), s])[0]
    xbuf = x.copy()
    sub = sess.submit(sess.host_bindings([xbuf, w.view(np.uint32), s]))
    xbuf[...] = 0  # scribble before the device has necessarily read anything
    assert sub.wait().output(3) == want


def test_each_submission_reports_its_own_status(dev):
    m, n, k = 1, 512, 4096
    x, w, s = synth.int4_linear_inputs(m, n, k, seed=12)
    sess = gemv_session(dev, m, n, k)
    bs = sess.host_bindings([x, w.view(np.uint32), s])
    want = sess.submit(bs).wait().output(3)
    a = sess.submit(bs)                                   # healthy, still to be waited for
    ffi.check(ffi.lib().vyb_instance_inject_status(sess.instance._h, 64))  # as if the NEXT kernel's bounded wait ran out
    b = sess.submit(bs)                                   # reads the raised word
    c = sess.submit(bs)                                   # healthy again: b cleared the word on the stream
    assert a.wait().output(3) == want                     # a is not blamed for b
    with pytest.raises(vb.BackendError, match="bounded device-side wait") as e:
        b.wait()
    assert e.value.code == ffi.ERR_DISPATCH_FAILED and "Fix:" in str(e.value)
    assert c.wait().output(3) == want                     # and b's failure does not leak into c


def test_prepared_submissions_equal_ordinary_ones(dev):
    m, n, k = 2, 777, 4096
    x, w, s = synth.int4_linear_inputs(m, n, k, seed=13)
    sess = gemv_session(dev, m, n, k)
    hw, hs = dev.resident_from(w.view(np.uint32)), dev.resident_from(s)
    bs = vb.BindingSet(sess.artifact.digest())
    bs.insert_host(0, x)
    bs.insert_resident(1, hw)
    bs.insert_resident(2, hs)
    want = sess.submit(bs).wait().output(3)
    prep = sess.prepare(bs)
    assert prep.submit().wait().output(3) == want          # replay with the prepared bytes
    x2, _, _ = synth.int4_linear_inputs(m, 16, k, seed=14)
    got2 = prep.submit({0: x2}).wait().output(3)            # new activations, same weights
    want2 = oracle.int4_rowmajor_linear(x2, w, s, m, n, k)
    assert np.array_equal(np.frombuffer(got2, np.uint16).reshape(m, n), want2)
    # one submission per prepared set in flight
    pending = prep.submit({0: x})
    with pytest.raises(vb.BackendError, match="has not been waited for"):
        prep.submit({0: x})
    done = pending.wait()
    assert done.output(3) == want
    with pytest.raises(vb.BackendError, match="has not been waited for"):
        prep.submit({0: x})                                 # the completion still views the set's buffers
    del done
    assert prep.submit({0: x}).wait().output(3) == want
    # wrong sizes and non-input ids are refused
    with pytest.raises(vb.BackendError, match="must be exactly"):
        prep.submit({0: x[:, : k // 2].copy()})
    with pytest.raises(vb.BackendError, match="not a host input"):
        prep.submit({1: w.view(np.uint32)})
    # the resident weights are held by the prepared set
    with pytest.raises(vb.BackendError, match="in-flight"):
        dev.free_resident(hw)
    with pytest.raises(vb.BackendError, match="in flight"):
        dev.upload_resident_at(hw, 0, np.zeros(4, np.uint32))
    prep.free()
    dev.free_resident(hw)
    dev.free_resident(hs)


@pytest.mark.parametrize("m,n,out_dtype", [(8, 4096, ffi.DT_F32),     # 128 KB: the kernel stores into the set's mapped host buffer
                                           (8, 14336, ffi.DT_F32),    # 448 KB: device buffer plus a copy node
                                           (40, 2048, ffi.DT_BF16)])  # the tensor-core path (batch > 8), 160 KB, direct
def test_prepared_outputs_direct_or_copied_equal_ordinary_submissions(dev, m, n, out_dtype):
    k = 4096
    x, w, s = synth.int4_linear_inputs(m, n, k, seed=21)
    prog = vb.linear_int4_grouped_rowmajor("x", "w", "scale", "out", m, k, n, 128, out_dtype)
    sess = vb.ArtifactSession.compile(prog, dev)
    hw, hs = dev.resident_from(w.view(np.uint32)), dev.resident_from(s)
    bs = vb.BindingSet(sess.artifact.digest())
    bs.insert_host(0, x)
    bs.insert_resident(1, hw)
    bs.insert_resident(2, hs)
    want = sess.submit(bs).wait().output(3)
    prep = sess.prepare(bs)
    for _ in range(3):  # replays reuse the same output buffer
        done = prep.submit({0: x}).wait()
        assert done.output(3) == want
        del done
    x2 = synth.int4_linear_inputs(m, 16, k, seed=22)[0]
    bs2 = vb.BindingSet(sess.artifact.digest())
    bs2.insert_host(0, x2)
    bs2.insert_resident(1, hw)
    bs2.insert_resident(2, hs)
    want2 = sess.submit(bs2).wait().output(3)
    done = prep.submit({0: x2}).wait()
    assert done.output(3) == want2 and want2 != want
    del done
    prep.free()
    dev.free_resident(hw)
    dev.free_resident(hs)
