"""Failures that must be seen and must leave everything usable: a kernel whose bounded wait runs out (made to
happen in the form the kernels provide for: a copy that is expected to bring more bytes than it does, with the
limit set to a few milliseconds; nothing traps, faults or waits without bound), and a device that has no room."""
import pytest
import torch

from gpu_util import DEV, check
from nncpu_b200 import Engine, ExtensionError, GenerateParams, Model, OutOfMemory, SamplerParams, Session, SessionParams
from nncpu_b200.kernels import ops
from nncpu_b200.parts import Runtime
from tiny import make_folder

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_sets_the_status_and_the_next_product_is_right():
    rt = Runtime(DEV, torch.bfloat16)
    ws = rt.workspace
    g = torch.Generator().manual_seed(0)
    x = torch.randn(128, 384, generator=g).bfloat16().to(DEV)      # six k-blocks through four stages: the
    w = (torch.randn(256, 384, generator=g) * 0.1).bfloat16().to(DEV)   # producer runs into its limit too
    out = torch.full((128, 256), 7.0, device=DEV)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    ops.linear_tc_wait_probe(x, w, out, ws, limit_ms=3)
    b.record()
    torch.cuda.synchronize()                                       # the kernel returned by itself
    assert 3.0 <= a.elapsed_time(b) < 200.0
    assert float(out.min()) == 7.0 and float(out.max()) == 7.0     # nothing half-done was stored
    assert int(ws.status.item()) in (101, 102, 103, 104)
    with pytest.raises(ExtensionError, match="gave up waiting"):
        rt.check_status()
    rt.check_status()                                              # the word is clear again
    # the same workspace, the same kernel, an ordinary product
    good = torch.full((300, 256), 9.0, device=DEV)
    x2 = torch.randn(300, 384, generator=g).bfloat16().to(DEV)
    ops.linear_tc(x2, w, None, good, ws, plan="never_even")
    check(good, (x2.double() @ w.double().T).float(), 1e-5, "the product after the probe")
    rt.check_status()


def test_generation_raises_when_a_kernel_gave_up_and_frees_its_slots(tmp_path):
    folder = make_folder(tmp_path / "m", "G", seed=2, store_dtype=torch.bfloat16)
    model = Model.load(folder, dtype="bfloat16")
    session = Session(model, SessionParams(n_ctx=128, seed=1, max_batch=2))
    ok = session.generate([[1, 2, 3], [4, 5]], GenerateParams(6, SamplerParams.greedy()), stop_token_ids=())
    ws = model.rt.workspace
    x = torch.zeros(128, 128, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(256, 128, dtype=torch.bfloat16, device=DEV)
    ops.linear_tc_wait_probe(x, w, torch.zeros(128, 256, device=DEV), ws, limit_ms=2)
    with pytest.raises(ExtensionError, match="gave up waiting"):
        session.generate([[1, 2, 3], [4, 5]], GenerateParams(6, SamplerParams.greedy()), stop_token_ids=())
    assert session.engine.cache.slots.n_held == 0
    session.engine.cache.check()
    again = session.generate([[1, 2, 3], [4, 5]], GenerateParams(6, SamplerParams.greedy()), stop_token_ids=())
    assert [r.tokens for r in again] == [r.tokens for r in ok]
    # the one-sequence calls look at the word too
    ops.linear_tc_wait_probe(x, w, torch.zeros(128, 256, device=DEV), ws, limit_ms=2)
    with pytest.raises(ExtensionError):
        session.eval([1, 2, 3])


def test_no_room_on_the_device_is_out_of_memory_with_the_sizes(tmp_path):
    folder = make_folder(tmp_path / "m", "A", seed=2)
    model = Model.load(folder, dtype="float32")
    free_before = torch.cuda.mem_get_info()[0]
    with pytest.raises(OutOfMemory, match=r"a cache of \d+ tokens .*GiB") as e:
        Engine(model, max_tokens=2 ** 31)           # 512 GiB of keys and values: one refused allocation
    assert e.value.kind == "OutOfMemory" and isinstance(e.value, MemoryError)
    assert torch.cuda.mem_get_info()[0] >= free_before - (64 << 20)
    # a step that runs out of room leaves the cache as it was
    engine = Engine(model, max_tokens=64 * 8)
    s = engine.alloc_slot()
    engine.step([s], [[1, 2, 3]])
    pages = engine.cache.groups[0].pool.n_free
    real = model.forward

    def no_room(ctx, cache):
        raise torch.OutOfMemoryError("CUDA out of memory. Tried to allocate 20.00 GiB. GPU 0 has ...")
    model.forward = no_room
    try:
        with pytest.raises(OutOfMemory, match="a step of 300 tokens in 1 sequences.*Tried to allocate 20.00 GiB"):
            engine.step([s], [[i % 200 for i in range(300)]])
        assert engine.cache.length(s) == 3 and engine.cache.groups[0].pool.n_free == pages
        # the same through the captured form of one sequence's short prompt step
        with pytest.raises(OutOfMemory, match="a prompt step of 200 tokens.*Tried to allocate 20.00 GiB"):
            engine.step([s], [list(range(200))])
    finally:
        model.forward = real
    assert engine.cache.length(s) == 3 and engine.cache.groups[0].pool.n_free == pages
    engine.cache.check()
    assert engine.step([s], [[4]]).shape == (1, 256)
