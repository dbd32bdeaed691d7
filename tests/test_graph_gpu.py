"""CUDA-graph replay of a fixed-shape forward pass (turbotransformers_b200/graphs.py) with the allocator in arena mode:
the replayed pass must reproduce the eager pass bit for bit on new inputs, and the arena must behave (fixed addresses, no
driver allocation, loud exhaustion)."""
import ctypes as C

import pytest
import torch

import turbotransformers_b200 as tt
from turbotransformers_b200 import _capi, synthetic
from turbotransformers_b200._cxx import cxx
from turbotransformers_b200.graphs import CapturedForward

pytestmark = pytest.mark.gpu
torch.set_grad_enabled(False)
DEV = torch.device("cuda:0")


@pytest.mark.parametrize("batch,seq", [(1, 128), (4, 64)])
def test_captured_bert_forward_replays_the_eager_pass(batch, seq):
    hf = synthetic.make_hf_bert("bert-mini", 7)
    model = tt.BertModel.from_torch(hf.to(DEV).half(), DEV)
    ids = [synthetic.random_ids(batch, seq, hf.config.vocab_size, s).to(DEV) for s in range(3)]
    eager = [tuple(t.clone() for t in model(i)[:2]) for i in ids]
    replay = CapturedForward(lambda x: model(x)[:2], ids[0].clone())
    assert 0 < replay.arena_used <= replay.arena_bytes
    for i, (seq_e, pooled_e) in zip(ids + ids[:1], eager + eager[:1]):  # new inputs, and the first one again
        seq_g, pooled_g = replay(i)
        torch.cuda.synchronize()
        assert torch.equal(seq_g, seq_e) and torch.equal(pooled_g, pooled_e)
    assert cxx.device_status(0) == 0
    # the eager path still works after a capture (the allocator is back on the pool)
    again = model(ids[1])[0]
    assert torch.equal(again, eager[1][0])


def test_two_captures_on_one_device_keep_their_own_buffers():
    hf = synthetic.make_hf_bert("bert-mini", 7)
    model = tt.BertModel.from_torch(hf.to(DEV).half(), DEV)
    small = [synthetic.random_ids(1, 32, hf.config.vocab_size, s).to(DEV) for s in range(2)]
    large = [synthetic.random_ids(4, 96, hf.config.vocab_size, s).to(DEV) for s in range(2)]
    eager_small = [model(i)[0].clone() for i in small]
    eager_large = [model(i)[0].clone() for i in large]
    first = CapturedForward(lambda x: model(x)[0], small[0].clone())
    second = CapturedForward(lambda x: model(x)[0], large[0].clone())   # a larger arena: the first one must survive it
    for k in (0, 1, 0):  # alternate between the two graphs
        out_small = first(small[k]).clone()
        out_large = second(large[k]).clone()
        torch.cuda.synchronize()
        assert torch.equal(out_small, eager_small[k]) and torch.equal(out_large, eager_large[k])
    second.close()
    assert torch.equal(first(small[1]), eager_small[1])   # releasing one leaves the other intact
    with pytest.raises(RuntimeError):
        second(large[0])
    first.close()
    assert cxx.device_status(0) == 0


def test_arena_mode_of_the_allocator(ctx):
    lib = _capi.lib()
    used = C.c_size_t(0)
    p1, p2, p3, a1, a2 = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_void_p()
    assert lib.ttb_arena_begin(ctx.h, 1 << 20) == _capi.OK
    assert lib.ttb_arena_begin(ctx.h, 1 << 20) == _capi.ERR_INVALID  # already active
    assert lib.ttb_alloc(ctx.h, 1000, b"a", C.byref(p1)) == _capi.OK
    assert lib.ttb_alloc(ctx.h, 5000, b"b", C.byref(p2)) == _capi.OK
    assert p2.value - p1.value == 1024  # 256-byte aligned, increasing
    assert lib.ttb_free(ctx.h, p1, b"a") == _capi.OK  # no-op
    assert lib.ttb_alloc(ctx.h, 2 << 20, b"too big", C.byref(p3)) == _capi.ERR_OOM
    assert lib.ttb_arena_end(ctx.h, C.byref(used), C.byref(a1)) == _capi.OK and used.value == 1024 + 5000
    assert a1.value == p1.value  # the handle is the buffer; its first block starts at offset 0
    assert lib.ttb_arena_end(ctx.h, None, None) == _capi.ERR_INVALID  # nothing active
    first = p1.value
    assert lib.ttb_arena_begin(ctx.h, 1 << 19) == _capi.OK  # a buffer of its own: the first arena may be in use by a graph
    assert lib.ttb_alloc(ctx.h, 64, b"c", C.byref(p2)) == _capi.OK
    assert not (first <= p2.value < first + (1 << 20))
    assert lib.ttb_arena_release(ctx.h, p2) == _capi.ERR_INVALID  # still active
    assert lib.ttb_arena_end(ctx.h, None, C.byref(a2)) == _capi.OK
    assert lib.ttb_free(ctx.h, p1, b"a") == _capi.OK and lib.ttb_free(ctx.h, p2, b"c") == _capi.OK  # no-ops after the arenas ended
    assert lib.ttb_alloc(ctx.h, 4096, b"pool", C.byref(p3)) == _capi.OK  # back on the pool
    assert not (first <= p3.value < first + (1 << 20))
    assert lib.ttb_free(ctx.h, p3, b"pool") == _capi.OK
    assert lib.ttb_arena_release(ctx.h, a1) == _capi.OK and lib.ttb_arena_release(ctx.h, a2) == _capi.OK
    assert lib.ttb_arena_release(ctx.h, a1) == _capi.ERR_INVALID  # already released
