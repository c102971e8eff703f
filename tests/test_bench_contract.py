"""The bench's JSON helpers on CPU: roofline denominators and fields, workload table."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_mod", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_roofline_uses_the_sustained_rate_for_a_seconds_long_loop_and_burst_otherwise():
    b = _bench()
    w = b.WORKLOADS["wan"]
    long_run = b.roofline(w, {"ms_per_step": 3900.0, "steps": 5}, 1200.0, 97.5, 1, 1680.8, 1396.3, "measured")
    assert long_run["peak"] == 1396.3 and abs(long_run["frac"] - 1200.0 / 1396.3) < 1e-12
    assert abs(long_run["frac_of_burst"] - 1200.0 / 1680.8) < 1e-12
    short = b.roofline(b.WORKLOADS["flux"], {"ms_per_step": 12.5, "steps": 5}, 1200.0, 0.22, 1, 1680.8, 1396.3,
                       "measured")
    assert short["peak"] == 1680.8 and "burst" in short["peak_kind"]
    for r in (long_run, short):
        assert r["bound"] == "tensor" and r["unit"] == "TFLOP/s" and r["kernel"] == "attn_fwd_sm100_kernel"
        assert r["traffic"] >= r["algorithmic_bytes"] > 0
    # traffic is per launch and per GPU: q, k, v read once, the output written once
    H, S, D = w["H"], w["S"], w["D"]
    assert long_run["algorithmic_bytes"] == 4 * H * S * D * 2


def test_workloads_match_the_named_configs():
    b = _bench()
    flux, wan = b.WORKLOADS["flux"], b.WORKLOADS["wan"]
    assert (flux["H"], flux["D"], flux["S"], flux["layers"]) == (24, 128, 4608, 57)
    assert (wan["H"], wan["D"], wan["S"], wan["layers"]) == (40, 128, 75600, 40)
    assert abs(b.flops_per_call(flux) - 2.609e11) / 2.609e11 < 1e-3
    assert abs(b.flops_per_call(wan) - 1.1705e14) / 1.1705e14 < 1e-3
    hun = b.WORKLOADS["hunyuan"]
    assert (hun["H"], hun["D"], hun["S"]) == (24, 128, 118800 + 256)
    for w in (flux, wan, hun):
        for n in (1, 2, 4, 8):  # Ulysses degree = ranks for flux/wan, ring degree = ranks for hunyuan
            assert w["S"] % n == 0 and (w is hun or w["H"] % n == 0)
    assert (b.TOL_MAX_ABS, b.TOL_COS) == (2e-2, 0.9999)


def test_nvlink_bytes_per_call():
    b = _bench()
    wan = b.WORKLOADS["wan"]
    # Ulysses 2 x ring 4: q,k,v and the output each move half of a local tensor; the ring sends the
    # K/V shard of 20 heads x 18,900 rows three times
    r = b.nvlink_bytes(wan, 2, 4)
    local = 40 * 9450 * 128 * 2
    assert r["ulysses_bytes_per_call"] == 4 * local / 2
    assert r["ring_bytes_per_call"] == 3 * 2 * 20 * 18900 * 128 * 2
    assert abs(r["ring_bytes_per_call"] - 580.6e6) / 580.6e6 < 1e-3
    assert b.nvlink_bytes(wan, 1, 1)["floor_ms_at_900GBs"] == 0.0
