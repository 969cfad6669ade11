"""The profiling module without a GPU: off it records nothing; host scopes add up."""
import io
import time

from pulsar_b200 import profiling


def test_off_by_default_and_scopes_cost_nothing():
    assert profiling.ENABLED is False
    with profiling.scope("x"), profiling.kernel("y"):
        pass
    assert profiling.totals() == ({}, {})
    out = io.StringIO()
    profiling.report(out)
    assert out.getvalue() == ""


def test_host_scopes_add_up(monkeypatch):
    monkeypatch.setattr(profiling, "ENABLED", True)
    try:
        for _ in range(3):
            with profiling.scope("plan"):
                time.sleep(0.002)
        with profiling.scope("pack"):
            pass
        kernels, host = profiling.totals()
        assert kernels == {} and host["plan"][0] == 3 and host["plan"][1] >= 0.005 and host["pack"][0] == 1
        out = io.StringIO()
        profiling.report(out)
        text = out.getvalue()
        assert "host time per phase" in text and "plan" in text and "device time" not in text
    finally:
        profiling._host_totals.clear()
