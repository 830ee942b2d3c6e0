"""The kernels with multicast operand loads are for processes that own one GPU: off by default, on only by
request, and locked off for good in a process that is one rank of several or that sets out to drive several
devices. All of this is host logic and runs without a GPU; every case runs in a fresh process because the
switch is process-wide."""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

from cuda_hgemm_b200 import build

ROOT = Path(__file__).resolve().parent.parent

PRELUDE = """
import ctypes, json, sys
sys.path.insert(0, %r)
from cuda_hgemm_b200 import _native, api
lib = _native.load()
def plan(variant, bn):
    p = _native.Plan(); p.variant, p.bn, p.tma_store = variant, bn, 1
    return p
def pick(M, N, K):
    p = api.select_plan_untuned(M, N, K)
    return [p.variant, p.bn]
def mcast_plan_status():
    return lib.b200_hgemm_plan_supported(16384, 16384, 16384, ctypes.byref(plan(_native.VARIANT_CTA2_MCAST, 512)))
out = {}
""" % str(ROOT)


def run_case(body, env_extra=None):
    env = {k: v for k, v in os.environ.items() if k not in ("WORLD_SIZE", "LOCAL_WORLD_SIZE", "B200_HGEMM_MULTICAST",
                                                             "B200_HGEMM_NO_MULTICAST")}
    env.update(env_extra or {})
    code = PRELUDE + textwrap.dedent(body) + "\nprint(json.dumps(out))\n"
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    import json

    return json.loads(r.stdout.strip().splitlines()[-1])


needs_companion = pytest.mark.skipif(not build.MULTICAST_SO.exists(),
                                     reason="libb200_hgemm_mc.so is not part of this run")


def test_off_by_default(native_lib):
    out = run_case("""
        out["state"] = lib.b200_hgemm_multicast_state()
        out["pick"] = pick(16384, 16384, 16384)
        out["explicit"] = mcast_plan_status()
    """)
    from cuda_hgemm_b200 import _native

    assert out["state"] == _native.MULTICAST_OFF
    assert out["pick"] == [_native.VARIANT_CTA2, 512]          # the same tiles on plain pairs
    assert out["explicit"] == _native.ERR_UNSUPPORTED


@needs_companion
def test_a_single_gpu_process_can_switch_it_on_and_off(native_lib):
    out = run_case("""
        out["on"] = lib.b200_hgemm_enable_multicast(1)
        out["state_on"] = lib.b200_hgemm_multicast_state()
        out["pick_on"] = pick(16384, 16384, 16384)
        out["explicit_on"] = mcast_plan_status()
        out["off"] = lib.b200_hgemm_enable_multicast(0)
        out["state_off"] = lib.b200_hgemm_multicast_state()
        out["pick_off"] = pick(16384, 16384, 16384)
    """)
    from cuda_hgemm_b200 import _native

    assert (out["on"], out["state_on"]) == (_native.OK, _native.MULTICAST_ON)
    assert out["pick_on"] == [_native.VARIANT_CTA2_MCAST, 512] and out["explicit_on"] == _native.OK
    assert (out["off"], out["state_off"]) == (_native.OK, _native.MULTICAST_OFF)
    assert out["pick_off"] == [_native.VARIANT_CTA2, 512]


@needs_companion
def test_the_environment_can_ask_for_it(native_lib):
    out = run_case('out["state"] = lib.b200_hgemm_multicast_state()', {"B200_HGEMM_MULTICAST": "1"})
    from cuda_hgemm_b200 import _native

    assert out["state"] == _native.MULTICAST_ON


@pytest.mark.parametrize("var", ["WORLD_SIZE", "LOCAL_WORLD_SIZE"])
def test_a_rank_of_several_can_never_switch_it_on(native_lib, var):
    out = run_case("""
        out["state"] = lib.b200_hgemm_multicast_state()
        out["enable"] = lib.b200_hgemm_enable_multicast(1)
        out["state_after"] = lib.b200_hgemm_multicast_state()
        out["pick"] = pick(16384, 16384, 16384)
        out["slab"] = pick(2048, 16384, 16384)
        out["explicit"] = mcast_plan_status()
    """, {var: "2", "B200_HGEMM_MULTICAST": "1"})
    from cuda_hgemm_b200 import _native

    assert out["state"] == out["state_after"] == _native.MULTICAST_LOCKED_OFF
    assert out["enable"] == _native.ERR_UNSUPPORTED
    assert out["pick"] == [_native.VARIANT_CTA2, 512]
    assert out["slab"][0] == _native.VARIANT_CTA2
    assert out["explicit"] == _native.ERR_UNSUPPORTED


def test_a_handle_on_several_devices_locks_it_off(native_lib):
    """b200_mg_create with two devices locks the switch even where the call itself then fails (no GPUs here):
    the intent to drive several GPUs is what counts."""
    out = run_case("""
        out["before"] = lib.b200_hgemm_enable_multicast(1)
        handle = ctypes.c_void_p()
        one = (ctypes.c_int * 1)(0)
        lib.b200_mg_create(one, 1, ctypes.byref(handle))          # a group of one does not lock
        out["state_one"] = lib.b200_hgemm_multicast_state()
        two = (ctypes.c_int * 2)(0, 1)
        out["create"] = lib.b200_mg_create(two, 2, ctypes.byref(handle))
        out["state"] = lib.b200_hgemm_multicast_state()
        out["enable"] = lib.b200_hgemm_enable_multicast(1)
        out["pick"] = pick(16384, 16384, 16384)
        out["explicit"] = mcast_plan_status()
    """)
    from cuda_hgemm_b200 import _native

    assert out["state_one"] in (_native.MULTICAST_OFF, _native.MULTICAST_ON)
    assert out["state"] == _native.MULTICAST_LOCKED_OFF
    assert out["enable"] == _native.ERR_UNSUPPORTED
    assert out["pick"] == [_native.VARIANT_CTA2, 512]
    assert out["explicit"] == _native.ERR_UNSUPPORTED
