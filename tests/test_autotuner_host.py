"""Host logic of the tile selector, mirroring the reference's unit tests
(src/autotuner.rs:1052-1150, src/empirical_autotune.rs:967-1156)."""
import ctypes as C
import os

import pytest

from y_b200 import _lib, runtime
from y_b200._lib import lib

F16, F32, BF16, FP8, INT4 = 0, 1, 2, 3, 4


def key(m, n, k, p, gpu):
    return _lib.take_string(lib.y_autotune_persist_key(m, n, k, p, gpu.encode()))


def u32(*v):
    return (C.c_uint32 * len(v))(*v)


def test_persist_key_separates_shape_precision_and_gpu():
    a, b = "NVIDIA GeForce RTX 4070 Ti SUPER", "NVIDIA B200"
    assert key(4096, 4096, 4096, F16, a) == "AUTOTUNE_F16_4096x4096x4096_NVIDIAGeForceRTX4070TiSUPER"
    assert key(4096, 4096, 4096, FP8, b) == "AUTOTUNE_FP8_4096x4096x4096_NVIDIAB200"
    assert key(4096, 4096, 4096, F16, a) != key(4096, 4096, 4096, F16, b)
    assert key(4096, 4096, 4096, F16, a) != key(4096, 4096, 4096, FP8, a)
    assert key(1, 4096, 4096, F16, a) != key(4096, 4096, 1, F16, a)
    assert key(8, 11008, 4096, INT4, b).startswith("AUTOTUNE_INT4_")
    assert "=" not in key(4096, 4096, 4096, F16, a)
    assert key(1, 1, 1, F16, "").endswith("_UnknownGPU")


def test_persisted_values_round_trip_and_reject_garbage():
    out = u32(*([0] * 7))
    assert lib.y_autotune_parse_persisted(b"128,64,32,2,2,3", out) == 0
    assert list(out) == [128, 64, 32, 2, 2, 3, 4]
    # a measured entry of the reference's own profile (.ysu_hw_profile:95)
    assert lib.y_autotune_parse_persisted(b"32,64,64,2,2,3", out) == 0 and out[6] == 4
    for bad in (b"128,64,32", b"", b"not,a,tile,at,all,here"):
        assert lib.y_autotune_parse_persisted(bad, out) != 0


def test_store_lookup_nearest_and_atomic_rewrite(tmp_path):
    prof = tmp_path / ".ysu_hw_profile"
    prof.write_text("GPU_NAME=NVIDIA B200\nSM_COUNT=148\n")
    lib.y_autotune_set_profile_path(str(prof).encode())
    try:
        gpu = b"NVIDIA B200"
        assert lib.y_autotune_store(4096, 4096, 4096, FP8, gpu, u32(128, 256, 128, 4, 1, 4)) == 0
        assert lib.y_autotune_store(4096, 4096, 4096, FP8, gpu, u32(128, 128, 128, 4, 1, 6)) == 0  # replace
        assert lib.y_autotune_store(512, 512, 512, FP8, gpu, u32(128, 64, 128, 4, 1, 8)) == 0
        text = prof.read_text()
        assert text.startswith("GPU_NAME=NVIDIA B200\nSM_COUNT=148\n")  # foreign lines survive
        assert text.count("AUTOTUNE_FP8_4096x4096x4096_NVIDIAB200=") == 1
        assert "AUTOTUNE_FP8_4096x4096x4096_NVIDIAB200=128,128,128,4,1,6\n" in text
        assert not os.path.exists(str(prof) + ".tmp")
        out, near = u32(*([0] * 7)), u32(0, 0, 0)
        assert lib.y_autotune_lookup(4096, 4096, 4096, FP8, gpu, out, near) == 1
        assert list(out)[:6] == [128, 128, 128, 4, 1, 6]
        # within 2x in every dimension: borrowed, and reported with the source shape
        assert lib.y_autotune_lookup(3000, 4096, 8192, FP8, gpu, out, near) == 2
        assert list(near) == [4096, 4096, 4096]
        # more than 2x away in one dimension: nothing to borrow
        assert lib.y_autotune_lookup(64, 4096, 4096, FP8, gpu, out, near) == 0
        # other GPU, other precision: separate namespaces
        assert lib.y_autotune_lookup(4096, 4096, 4096, FP8, b"NVIDIA H100", out, near) == 0
        assert lib.y_autotune_lookup(4096, 4096, 4096, F16, gpu, out, near) == 0
        # a borrowed tile must be launchable at the requested K
        assert lib.y_autotune_lookup(4096, 4096, 4100, FP8, gpu, out, near) == 0
    finally:
        lib.y_autotune_set_profile_path(b"")
        lib.y_autotune_clear_cache()


def test_resolution_order(tmp_path, monkeypatch):
    prof = tmp_path / "profile"
    prof.write_text("AUTOTUNE_FP8_2048x2048x2048_NVIDIAB200=128,64,128,4,1,8\n")
    lib.y_autotune_set_profile_path(str(prof).encode())
    try:
        lib.y_autotune_clear_cache()
        lib.y_autotune_set_mode(0)  # cached: persisted entry wins over the analytic score
        assert runtime.autotune_select_config(2048, 2048, 2048, True)["cta_n"] == 64
        lib.y_autotune_clear_cache()
        lib.y_autotune_set_mode(1)  # analytic: the cache file is ignored
        assert runtime.autotune_select_config(2048, 2048, 2048, True)["cta_n"] == 256
        monkeypatch.setenv("Y_CTA_OVERRIDE", "128,128,128,4,1,6")  # override beats everything
        assert runtime.autotune_select_config(2048, 2048, 2048, True)["cta_n"] == 128
        monkeypatch.setenv("Y_CTA_OVERRIDE", "garbage")
        assert runtime.autotune_select_config(2048, 2048, 2048, True)["cta_n"] == 256
        monkeypatch.delenv("Y_CTA_OVERRIDE")
        monkeypatch.setenv("Y_AUTOTUNE", "cached")  # the environment overrides the process mode
        lib.y_autotune_clear_cache()
        assert runtime.autotune_select_config(2048, 2048, 2048, True)["cta_n"] == 64
    finally:
        lib.y_autotune_set_mode(0)
        lib.y_autotune_set_profile_path(b"")
        lib.y_autotune_clear_cache()


def test_launchability_follows_the_kernels_contract():
    assert lib.y_autotune_is_launchable(u32(128, 256, 128, 4, 1, 4), 4096, FP8)
    assert lib.y_autotune_is_launchable(u32(128, 64, 128, 4, 1, 8), 4096 + 16, FP8)  # K tail is zero-filled
    assert not lib.y_autotune_is_launchable(u32(128, 256, 128, 4, 1, 4), 4100, FP8)  # K % 16
    assert not lib.y_autotune_is_launchable(u32(64, 64, 64, 2, 2, 3), 4096, FP8)     # an sm_89 tile
    assert not lib.y_autotune_is_launchable(u32(128, 256, 128, 0, 1, 4), 4096, FP8)
    assert lib.y_autotune_is_launchable(u32(256, 256, 128, 4, 1, 6), 4096, FP8)      # CTA pair
    assert not lib.y_autotune_is_launchable(u32(256, 128, 128, 4, 1, 6), 4096, FP8)  # the pair has one shape
    assert lib.y_autotune_is_launchable(u32(8, 16, 1024, 8, 1, 20), 4096, INT4)
    assert not lib.y_autotune_is_launchable(u32(8, 16, 1024, 8, 1, 20), 4000, INT4)


def test_analytic_score_prefers_wide_tiles_unless_the_grid_starves():
    big = [lib.y_autotune_score(u32(128, n, 128, 4, 1, 4), 8192, 8192, 8192, FP8) for n in (256, 128, 64)]
    assert big[0] > big[1] > big[2]
    small = [lib.y_autotune_score(u32(128, n, 128, 4, 1, 4), 256, 256, 256, FP8) for n in (256, 128, 64)]
    assert small[2] > small[0]
    # the CTA-pair tile halves the A traffic again: it wins where the grid is full, and
    # is not offered where its second CTA would only multiply padding
    pair = u32(256, 256, 128, 4, 1, 6)
    assert lib.y_autotune_score(pair, 8192, 8192, 8192, FP8) > big[0]
    assert runtime.autotune_select_config(8192, 8192, 8192, True)["cta_m"] == 256
    assert runtime.autotune_select_config(128, 8192, 8192, True)["cta_m"] == 128


def rows(*r):
    flat = [float(x) for row in r for x in row]
    return (C.c_double * len(flat))(*flat), len(r)


def test_tie_break_prefers_warps_then_k_depth_but_never_overrides_a_real_gap():
    # real timings from the reference's test (src/empirical_autotune.rs:1081-1122)
    arr, n = rows((16, 32, 32, 1, 1, 4, 56.10, 56.81), (32, 64, 64, 2, 2, 3, 56.64, 57.08),
                  (32, 64, 32, 2, 2, 4, 56.91, 59.59))
    assert lib.y_autotune_select_winner(arr, n) == 1
    arr, n = rows((64, 64, 64, 2, 2, 3, 9.72, 9.80), (128, 128, 32, 4, 4, 2, 9.97, 9.98))
    assert lib.y_autotune_select_winner(arr, n) == 0
    arr, n = rows((32, 64, 32, 2, 2, 4, 56.53, 58.00), (32, 64, 64, 2, 2, 3, 56.60, 58.10))
    assert lib.y_autotune_select_winner(arr, n) == 1
    # identical structure: deterministic (:1124-1137)
    arr, n = rows((64, 128, 32, 2, 2, 3, 34.44, 35.13), (128, 64, 32, 2, 2, 3, 34.60, 35.20))
    assert lib.y_autotune_select_winner(arr, n) == lib.y_autotune_select_winner(arr, n)
    assert lib.y_autotune_select_winner(None, 0) == 0


def test_tie_band_tracks_the_regimes_noise_floor():
    # src/empirical_autotune.rs:1139-1150
    assert not lib.y_autotune_tied(9.72, 9.80, 9.97, 9.98)
    assert lib.y_autotune_tied(56.10, 57.71, 57.56, 59.00)
    assert lib.y_autotune_tied(10.0, 10.0, 10.02, 10.02)       # 0.25% floor
    assert not lib.y_autotune_tied(10.0, 10.0, 10.05, 10.05)


def test_weight_replication_defeats_l2_only_where_it_has_to():
    # src/empirical_autotune.rs:1041-1065, with the reference's 48 MB L2 ...
    L2, plenty = 50_331_648, 14 << 30
    b = 4096 * 4096 * 2
    n = lib.y_autotune_plan_weight_replicas(b, 4096 * 2, 4096 * 4, L2, plenty)
    assert n >= 6 and b * n >= L2 * 4
    big = 16384 * 16384 * 2
    assert lib.y_autotune_plan_weight_replicas(big, big, 16384 * 16384 * 4, L2, plenty) == 1
    assert lib.y_autotune_plan_weight_replicas(b, 0, 0, L2, 40 << 20) == 1
    assert lib.y_autotune_plan_weight_replicas(b, 0, 0, 0, plenty) == 1
    # ... and with B200's: the 23 MB INT4 stream needs more than the reference's cap of 8 copies
    l2_b200 = 126 << 20
    stream = lib.y_b200_int4_stream_bytes(4096, 11008)
    n = lib.y_autotune_plan_weight_replicas(stream, 8 * 4096 * 2, 8 * 11008 * 2, l2_b200, 170 << 30)
    assert n > 8 and stream * n >= 4 * l2_b200
