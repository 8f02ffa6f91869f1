"""Host-side rules of the scratch-reusing int4 wrappers (vyre-self-substrate/src/math/quantized_dispatch/*.rs): the shape
checks and their `Fix:` texts run before anything is dispatched, so they are tested without a device, like the reference
tests them against a dispatcher that is never reached. DispatchError kinds map to status codes 2001-2003 and the messages
carry the reference's Display prefixes (optimizer/dispatcher.rs:112-120)."""
import numpy as np
import pytest

import vyre_b200 as vb
from vyre_b200 import ffi


@pytest.fixture()
def scratch():
    s = vb.QuantizedScratch(None)
    yield s
    s.close()


def bad(fn, *args):
    with pytest.raises(vb.BackendError) as e:
        fn(*args)
    return e.value


def test_unpack_rejects_zero_lanes_and_wrong_word_count(scratch):
    e = bad(vb.unpack_i4x8_via, scratch, np.zeros(1, np.uint32), 0)
    assert e.code == ffi.ERR_DISPATCH_BAD_INPUTS
    assert e.message == "dispatcher input mismatch: Fix: unpack_i4x8_via requires lane_count > 0."
    e = bad(vb.unpack_i4x8_via, scratch, np.zeros(3, np.uint32), 9)
    assert e.message == ("dispatcher input mismatch: Fix: unpack_i4x8_via requires packed_words.len() == "
                         "i4_packed_words(lane_count), got len=3 expected=2 for lane_count=9.")


def test_dot_rejects_mismatched_lengths(scratch):
    e = bad(vb.i4x8_dot_f32_scaled_via, scratch, np.zeros(1, np.uint32), np.zeros(2, np.uint32), 1.0, 1.0, 16)
    assert e.code == ffi.ERR_DISPATCH_BAD_INPUTS
    assert e.message == ("dispatcher input mismatch: Fix: i4x8_dot_f32_scaled_via requires lhs/rhs packed lengths == "
                         "i4_packed_words(lane_count), got lhs=1 rhs=2 expected=2 for lane_count=16.")
    assert "requires lane_count > 0" in bad(vb.i4x8_dot_f32_scaled_via, scratch, [], [], 1.0, 1.0, 0).message


def test_matvec_shape_rules(scratch):
    w = np.zeros(3 * 2, np.uint32)
    e = bad(vb.i4x8_matvec_f32_scaled_via, scratch, w, np.zeros(9, np.float32), np.zeros(3, np.float32), 0, 9)
    assert e.message == "dispatcher input mismatch: Fix: i4x8_matvec_f32_scaled_via requires rows > 0 and cols > 0, got rows=0 cols=9."
    e = bad(vb.i4x8_matvec_f32_scaled_via, scratch, w[:5], np.zeros(9, np.float32), np.zeros(3, np.float32), 3, 9)
    assert e.message.endswith("requires weights_packed.len() == rows*i4_packed_words(cols), got len=5 expected=6 for rows=3 cols=9.")
    e = bad(vb.i4x8_matvec_f32_scaled_via, scratch, w, np.zeros(8, np.float32), np.zeros(3, np.float32), 3, 9)
    assert e.message.endswith("requires x.len() == cols, got len=8 cols=9.")
    e = bad(vb.i4x8_matvec_f32_scaled_via, scratch, w, np.zeros(9, np.float32), np.zeros(2, np.float32), 3, 9)
    assert e.message.endswith("requires row_scales.len() == rows, got len=2 rows=3.")


def test_batched_matvec_shape_rules(scratch):
    w = np.zeros(3 * 2, np.uint32)
    e = bad(vb.i4x8_batched_matvec_f32_scaled_via, scratch, w, np.zeros(18, np.float32), np.zeros(3, np.float32), 0, 3, 9)
    assert e.message.endswith("requires batch > 0, rows > 0, and cols > 0, got batch=0 rows=3 cols=9.")
    e = bad(vb.i4x8_batched_matvec_f32_scaled_via, scratch, w, np.zeros(17, np.float32), np.zeros(3, np.float32), 2, 3, 9)
    assert e.message.endswith("requires x_batches.len() == batch*cols, got len=17 expected=18 for batch=2 cols=9.")


@pytest.mark.parametrize("fn,ctx", [(vb.i4x8_batched_matmul_f32_scaled_via, "i4x8_batched_matmul_f32_scaled_via"),
                                    (vb.i4x8_batched_matmul_top1_f32_scaled_via, "i4x8_batched_matmul_top1_f32_scaled_via")])
def test_batched_matmul_shape_rules(scratch, fn, ctx):
    w, a, rs, bs = np.zeros(6, np.uint32), np.zeros(4, np.uint32), np.zeros(3, np.float32), np.zeros(2, np.float32)
    assert bad(fn, scratch, w, a, rs, bs, 2, 3, 0).message == (
        f"dispatcher input mismatch: Fix: {ctx} requires batch > 0, rows > 0, and cols > 0, got batch=2 rows=3 cols=0.")
    assert bad(fn, scratch, w, a[:3], rs, bs, 2, 3, 9).message.endswith(
        "requires activation_batches_packed.len() == batch*i4_packed_words(cols), got len=3 expected=4 for batch=2 cols=9.")
    assert bad(fn, scratch, w, a, rs, bs[:1], 2, 3, 9).message.endswith("requires batch_scales.len() == batch, got len=1 batch=2.")
    assert bad(fn, scratch, w, a, rs[:2], bs, 2, 3, 9).message.endswith("requires row_scales.len() == rows, got len=2 rows=3.")


def test_valid_shapes_reach_the_dispatcher_and_a_scratch_without_device_rejects(scratch):
    e = bad(vb.unpack_i4x8_via, scratch, np.zeros(2, np.uint32), 9)
    assert e.code == ffi.ERR_DISPATCH_REJECTED and e.message.startswith("dispatcher rejected program: Fix:")
    assert scratch.stats() == {"cached": 0, "hits": 0, "misses": 1}
