"""The NVLink probe against a FAKE NVML (a shared object built by the test), the import
diagnosis and the doctor CLI. No GPU needed."""

import io
import subprocess
import textwrap

import pytest

import fast_ulysses_b200 as fu
from fast_ulysses_b200.utils import cli, diagnose

FAKE = textwrap.dedent(r"""
    #include <string.h>
    #include <stdlib.h>
    // A 4-GPU machine: 0,1,2 hang off one NVSwitch; 3 has a direct link to 0 only; link 5 of GPU 2 is down.
    typedef struct { char legacy[16]; unsigned domain, bus, device, id, sub; char bus_id[32]; } pci_t;
    static const char* ids[4] = {"00000000:1B:00.0", "00000000:2C:00.0", "00000000:3D:00.0", "00000000:4E:00.0"};
    int nvmlInit_v2(void) { return getenv("FAKE_NVML_FAIL_INIT") ? 1 : 0; }
    int nvmlDeviceGetHandleByPciBusId_v2(const char* bus, void** dev) {
        for (long i = 0; i < 4; ++i) {
            size_t n = strlen(bus), m = strlen(ids[i]);
            if (strcasecmp(bus + (n > 12 ? n - 12 : 0), ids[i] + (m - 12)) == 0) { *dev = (void*)(i + 1); return 0; }
        }
        return 2;
    }
    int nvmlDeviceGetNvLinkState(void* dev, unsigned link, unsigned* active) {
        long g = (long)dev - 1;
        *active = (link < 2) && !(g == 2 && link == 1);
        return link < 18 ? 0 : 3;
    }
    int nvmlDeviceGetNvLinkRemoteDeviceType(void* dev, unsigned link, int* kind) {
        long g = (long)dev - 1;
        *kind = (g == 3 || (g == 0 && link == 1)) ? 0 : 2;  // 0 = GPU, 2 = switch
        return 0;
    }
    int nvmlDeviceGetNvLinkRemotePciInfo_v2(void* dev, unsigned link, pci_t* out) {
        long g = (long)dev - 1;
        memset(out, 0, sizeof(*out));
        strcpy(out->bus_id, g == 3 ? ids[0] : ids[3]);
        return 0;
    }
""")
IDS = ["0000:1b:00.0", "0000:2c:00.0", "0000:3d:00.0", "0000:4e:00.0"]


@pytest.fixture()
def fake_nvml(tmp_path):
    src = tmp_path / "fake_nvml.c"
    lib = tmp_path / "libfake_nvml.so"
    src.write_text("#include <strings.h>\n" + FAKE)
    subprocess.run(["gcc", "-shared", "-fPIC", "-o", str(lib), str(src)], check=True)
    fu._C._set_nvml_library(str(lib))
    yield lib
    fu._C._set_nvml_library("")


def test_matrix_from_fake_nvml(fake_nvml):
    m = fu._C._nvlink_matrix_by_bus_id(IDS, [0, 1, 2, 3])
    assert m is not None and len(m) == 12
    for i, j in ((0, 1), (1, 0), (0, 2), (2, 1)):
        assert m[(i, j)], (i, j)          # one switch fabric
    assert m[(0, 3)] and m[(3, 0)]         # direct link
    assert not m[(1, 3)] and not m[(3, 2)]  # 3 is not on the switch


def test_unknown_device_fails_open(fake_nvml):
    assert fu._C._nvlink_matrix_by_bus_id(IDS[:2] + ["0000:99:00.0"], [0, 1, 2]) is None


def test_missing_nvml_fails_open():
    fu._C._set_nvml_library("/nonexistent/libnvidia-ml.so.1")
    try:
        assert fu._C._nvlink_matrix_by_bus_id(IDS, [0, 1, 2, 3]) is None
        assert fu.nvlink_matrix([0, 999]) is None
        assert fu._C.check_nvlink([0, 999]) == ""
    finally:
        fu._C._set_nvml_library("")


def test_import_diagnosis_names_the_mismatch():
    live = diagnose.live_facts()
    built = dict(live, torch="2.9.0")
    msg = diagnose.verdict("undefined symbol: _ZN3c10", built, live)
    assert "built against torch 2.9.0" in msg
    assert "CUDA" in diagnose.verdict("libcudart.so.12: cannot open shared object file", live, live)
    assert "rebuild" in diagnose.verdict("something else", live, live)


def test_doctor_runs_without_a_gpu():
    buf = io.StringIO()
    rc = cli.doctor(out=buf)
    text = buf.getvalue()
    assert "fast_ulysses_b200" in text and "sm_100a" in text and "devices" in text
    assert rc in (0, 1)
