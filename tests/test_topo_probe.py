"""NVLink attribute probe against a fake management library (built here with gcc): the real one needs a GPU driver."""
import ctypes as C
import json
import os
import subprocess
import sys

import pytest

from cann_hccl_b200 import _lib as L

FAKE = r"""
#include <string.h>
static int n_links = %(links)d, n_down = %(down)d, version = %(version)d, speed = %(speed)d;
int nvmlInit_v2(void) { return 0; }
int nvmlDeviceGetHandleByIndex_v2(unsigned i, void **d) { *d = (void *)(long)(i + 1); return i < 8 ? 0 : 2; }
int nvmlDeviceGetName(void *d, char *n, unsigned len) { strncpy(n, "FAKE B200", len); return 0; }
int nvmlDeviceGetNvLinkState(void *d, unsigned l, unsigned *a) { if ((int)l >= n_links) return 2; *a = (int)l >= n_down; return 0; }
int nvmlDeviceGetNvLinkVersion(void *d, unsigned l, unsigned *v) { *v = version; return 0; }
int nvmlDeviceGetNvLinkRemoteDeviceType(void *d, unsigned l, unsigned *t) { *t = 1; return 0; }
struct fv { unsigned id, scope; long long ts, lat; unsigned type, ret; union { double d; unsigned ui; unsigned long long ull; } v; };
int nvmlDeviceGetFieldValues(void *d, int n, struct fv *f) { f->ret = speed ? 0 : 3; f->v.ui = speed; return 0; }
"""


def probe(tmp_path, name, **kw):
    src = tmp_path / (name + ".c")
    so = tmp_path / ("lib" + name + ".so")
    src.write_text(FAKE % kw)
    subprocess.check_call(["gcc", "-shared", "-fPIC", "-o", str(so), str(src)])
    code = ("import ctypes as C, sys; sys.path.insert(0, %r); from cann_hccl_b200 import _lib as L; b = C.create_string_buffer(2048); "
            "lib = L.lib(); lib.HcclB200ProbeLinks.argtypes = [C.c_int32, C.c_char_p, C.c_size_t]; "
            "assert lib.HcclB200ProbeLinks(0, b, 2048) == 0; print(b.value.decode())") % os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, HCCL_NVML_LIB=str(so))
    out = subprocess.check_output([sys.executable, "-c", code], env=env, text=True)
    return json.loads(out.strip().splitlines()[-1])


def test_b200_like_device(tmp_path):
    t = probe(tmp_path, "b200", links=18, down=0, version=7, speed=0)
    assert t["probed"] and t["links_active"] == 18 and t["links_to_switch"] == 18 and t["nvswitch"]
    assert t["nvlink_version"] == 7 and t["link_gbps_per_direction"] == 50 and t["egress_gbps"] == 900


def test_links_down_and_reported_speed(tmp_path):
    t = probe(tmp_path, "h100", links=18, down=2, version=6, speed=26562)
    assert t["links_total"] == 18 and t["links_active"] == 16
    assert abs(t["link_gbps_per_direction"] - 26.562) < 1e-6 and abs(t["egress_gbps"] - 16 * 26.562) < 1e-3


def test_library_absent(tmp_path):
    code = ("import ctypes as C, sys; sys.path.insert(0, %r); from cann_hccl_b200 import _lib as L; b = C.create_string_buffer(2048); "
            "lib = L.lib(); lib.HcclB200ProbeLinks.argtypes = [C.c_int32, C.c_char_p, C.c_size_t]; "
            "assert lib.HcclB200ProbeLinks(0, b, 2048) == 0; print(b.value.decode())") % os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.check_output([sys.executable, "-c", code], env=dict(os.environ, HCCL_NVML_LIB=str(tmp_path / "nope.so")), text=True)
    t = json.loads(out.strip().splitlines()[-1])
    assert t["probed"] is False and t["links_active"] == 0
