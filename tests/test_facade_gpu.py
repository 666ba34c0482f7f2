"""Builds and runs the C++ facade test program (tests/facade_test.cu) against the shared library."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_facade_program(built_lib, tmp_path):
    exe = str(tmp_path / "facade_test")
    libdir = os.path.join(ROOT, "clusternet_b200")
    subprocess.check_call(["/usr/local/cuda/bin/nvcc", "-std=c++17", "-O1", "-gencode", "arch=compute_100a,code=sm_100a",
                           os.path.join(ROOT, "tests", "facade_test.cu"), "-o", exe, f"-L{libdir}", "-lclusternet_b200",
                           "-Xlinker", f"-rpath={libdir}"])
    r = subprocess.run([exe, os.path.join(ROOT, "tests", "golden", "codebook_126.f32"), str(tmp_path),
                        os.path.join(ROOT, "tests", "golden", "numpy_arange_as_h5py.hdf5"),
                        os.path.join(ROOT, "tests", "golden", "scipy_sparse_arange_as_h5py.hdf5")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "All tests passed" in r.stdout, r.stdout + r.stderr


def _build(tmp_path, name):
    exe = str(tmp_path / name)
    libdir = os.path.join(ROOT, "clusternet_b200")
    subprocess.check_call(["/usr/local/cuda/bin/nvcc", "-std=c++17", "-O1", "-gencode", "arch=compute_100a,code=sm_100a",
                           os.path.join(ROOT, "tests", name + ".cu"), "-o", exe, f"-L{libdir}", "-lclusternet_b200",
                           "-Xlinker", f"-rpath={libdir}"])
    return exe


def _run_ranks(exe, tmp_path, nranks):
    """One process per GPU, the way a launcher would start the reference's MPI program."""
    base = dict(os.environ, CN_CODEBOOK=os.path.join(ROOT, "tests", "golden", "codebook_126.f32"), NCCL_NVLS_ENABLE="0",
                WORLD_SIZE=str(nranks), CN_NCCL_ID_FILE=str(tmp_path / f"nccl_id_{nranks}"))
    procs = [subprocess.Popen([exe, str(tmp_path)], env=dict(base, RANK=str(r), LOCAL_RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(nranks)]
    # a rank that fails leaves the others waiting in their next collective: stop them soon after, and bound the whole run
    import time
    deadline = time.time() + 240
    failed_at = None
    while any(p.poll() is None for p in procs) and time.time() < deadline:
        if failed_at is None and any(p.poll() not in (None, 0) for p in procs):
            failed_at = time.time()
        if failed_at is not None and time.time() - failed_at > 10:
            break
        time.sleep(0.2)
    outs = []
    for p in procs:
        if p.poll() is None:
            p.kill()
        out, _ = p.communicate()
        outs.append((p.returncode, out))
    return outs


@pytest.mark.parametrize("program", ["readme_test", "batch_test"])
def test_reference_style_program_one_process(built_lib, tmp_path, program):
    exe = _build(tmp_path, program)
    for code, out in _run_ranks(exe, tmp_path, 1):
        assert code == 0 and "All tests passed" in out, out[-3000:]


@pytest.mark.parametrize("program", ["readme_test", "batch_test"])
def test_reference_style_program_one_process_per_gpu(built_lib, tmp_path, program):
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    exe = _build(tmp_path, program)
    outs = _run_ranks(exe, tmp_path, min(n, 4))
    report = "\n".join(f"[rank {r}: exit {code}] {out[-1500:]}" for r, (code, out) in enumerate(outs))
    assert all(code == 0 and "All tests passed" in out for code, out in outs), report


def test_several_gpus_in_one_process(built_lib, tmp_path):
    """cn_comm_init_all: ranks as contexts of one process, driven by one thread each and by a single thread with
    cn_group_start / cn_group_end (tests/initall_test.cu)."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    exe = _build(tmp_path, "initall_test")
    r = subprocess.run([exe, os.path.join(ROOT, "tests", "golden", "codebook_126.f32")], capture_output=True, text=True, timeout=300,
                       env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0 and "All tests passed" in r.stdout, r.stdout[-3000:] + r.stderr[-2000:]
