"""The phase profiler's bookkeeping and its report, fed with made-up timings (no GPU)."""
from nncpu_b200 import perf


def setup_function(_):
    perf.perf_enable(False)
    perf.perf_reset()


def test_report_without_samples():
    assert perf.perf_report("reply") == "nncpu perf (reply): no samples\n"


def test_report_table_from_fake_timings():
    # 2 ms of q/k/v products that streamed 10 GB and did 4 TFLOP; 1 ms of attention over 3 GB; norms count no bytes
    perf.add("attn_qkv", 1.0e6, 5e9, 2e12)
    perf.add("attn_qkv", 1.0e6, 5e9, 2e12)
    perf.add("attn_core", 1.0e6, 3e9, 0.2e12)
    perf.add("norm", 0.5e6)
    perf.add("moe_route", 0.5e6)          # a slot the library does not know joins after the known ones
    text = perf.perf_report("reply", n_tokens=8, peaks={"hbm_gbs": 6552.0, "bf16_tflops": 1628.5})
    lines = text.splitlines()
    assert lines[0].startswith("nncpu perf - reply") and "kernel by kernel" in lines[0]
    assert lines[1].split() == ["phase", "ms", "%", "calls", "us/call", "GB/s", "TFLOP/s", "of", "peak"]
    rows = {ln.split()[0]: ln.split() for ln in lines[3:]}
    assert list(rows)[:4] == ["norm", "attn_qkv", "attn_core", "moe_route"]       # forward order, then new slots
    assert rows["attn_qkv"][1:5] == ["2.0", "50.0%", "2", "1000.0"]
    assert rows["attn_qkv"][5:] == ["5000.0", "2000.0", "1.23", "mma"]           # 2000 / 1628.5 beats 5000 / 6552
    assert rows["attn_core"][5:] == ["3000.0", "200.0", "0.46", "hbm"]
    assert rows["norm"] == ["norm", "0.5", "12.5%", "1", "500.0"]                # no bytes: no rate columns
    assert rows["TOTAL"][1:] == ["4.0", "100.0%"]
    assert "memory traffic: 12.11 GB @ 3250.0 GB/s effective" in text
    assert "0.50 ms/token over 8 tokens" in text
    totals = perf.perf_totals()
    assert totals["attn_qkv"] == {"ms": 2.0, "calls": 2, "bytes": 1e10, "flops": 4e12}
    perf.perf_reset()
    assert perf.perf_totals() == {}


def test_scopes_are_free_when_off_and_pausable():
    assert not perf.enabled()
    assert perf.scope("norm") is perf._NULL                # off: the shared do-nothing scope, no event made
    with perf.scope("norm"):
        pass
    assert perf.perf_totals() == {}
    perf._on = True                                        # on without touching the device
    try:
        assert perf.enabled()
        with perf.paused():
            assert not perf.enabled() and perf.scope("norm") is perf._NULL
            with perf.paused():
                assert not perf.enabled()
            assert not perf.enabled()
        assert perf.enabled()
    finally:
        perf._on = False
