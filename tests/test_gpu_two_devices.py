"""One process driving two devices (the reference's multi-device model is one Network per device_id,
shadow/core/context.cu:10-15): per-device state of the kernel library - the opt-in to large dynamic
shared memory, the cached multiprocessor count, the built-in reduction scratch - must be set up on
each device it is used on.  Skipped on a machine with one GPU."""
import numpy as np
import pytest

import cases

pytestmark = pytest.mark.gpu


def test_kernels_with_per_device_state_run_on_a_second_device():
    import torch
    from shadow_b200 import capi
    from shadow_b200 import functional as F
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    x_soft = cases.normal(8100, (300, 1000, 7, 7), 0.0, 2.0)       # resident-plane Softmax (226 KB of shared memory)
    x_gn = cases.normal(8101, (40, 8, 56, 56))                     # GroupNorm over 100 KB rows staged in shared memory
    x_red = cases.normal(8102, (600, 64, 14, 14))                  # inner-kept Reduce with its copy ring
    want_soft = cases.run_port({"name": "s", "op": "Softmax", "args": {"axis": 1}, "inputs": [x_soft]})
    want_gn = cases.run_port({"name": "g", "op": "GroupNorm", "args": {"group": 1, "eps": 1e-5}, "inputs": [x_gn]})
    want_red = cases.run_port({"name": "r", "op": "Reduce", "args": {"operation": 1, "axes": [1], "keep_dims": True}, "inputs": [x_red]})
    for dev in (0, 1, 0):
        with torch.cuda.device(dev):
            d = torch.device("cuda", dev)
            got_soft = F.softmax(torch.from_numpy(x_soft).to(d), 1)
            got_gn = F.group_norm(torch.from_numpy(x_gn).to(d), 1, None, None, 1e-5)
            got_red = F.reduce(torch.from_numpy(x_red).to(d), 1, [1], keep_dims=True)
            lib = capi.lib()
            y = torch.empty(1, device=d)
            big = torch.from_numpy(cases.normal(8103, (8, 1024, 1024))).to(d)
            capi.check(lib.sb200_reduce_static(big.data_ptr(), capi.ints(big.shape), 3, capi.ints([0, 1, 2]), 3, 1, y.data_ptr(),
                                               torch.cuda.current_stream().cuda_stream), "sb200_reduce_static")
            torch.cuda.synchronize()
            assert lib.sb200_softmax_ring_timeouts() == 0
            cases.assert_parity({"name": "s", "op": "Softmax", "args": {"axis": 1}, "inputs": [x_soft]}, got_soft.cpu().numpy(), want_soft)
            cases.assert_parity({"name": "g", "op": "GroupNorm", "args": {"group": 1, "eps": 1e-5}, "inputs": [x_gn]},
                                got_gn.cpu().numpy().reshape(want_gn.shape), want_gn)
            cases.assert_parity({"name": "r", "op": "Reduce", "args": {"operation": 1, "axes": [1], "keep_dims": True}, "inputs": [x_red]},
                                got_red.cpu().numpy().reshape(want_red.shape), want_red)
            assert np.isclose(float(y.item()), float(np.sum(big.cpu().numpy().astype(np.float64))), rtol=1e-5, atol=1e-2)


def test_cpp_host_with_one_thread_per_device_uses_the_c_entry_points(tmp_path):
    """tests/support/comm_two_threads.cpp: no Python in the data path - a C++ program whose two host threads
    each own a device, shard a tensor, and finish a Sum and a Max over all axes with one
    sb200_sharded_reduce_finish call."""
    import os
    import shutil
    import subprocess
    import torch
    from shadow_b200 import build as sbuild
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    if sbuild.build_comm() is None:
        pytest.skip("no NCCL on this machine")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    lib_dir = os.path.join(root, "shadow_b200", "lib")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cuda_home = os.path.dirname(os.path.dirname(nvcc))
    exe = str(tmp_path / "comm_two_threads")
    build = subprocess.run(["g++", "-O1", "-std=c++17", "-o", exe, os.path.join(root, "tests", "support", "comm_two_threads.cpp"),
                            "-I" + os.path.join(root, "include"), "-I" + os.path.join(cuda_home, "include"),
                            "-L" + lib_dir, "-lsb200_nccl", "-lsb200", "-Wl,-rpath," + lib_dir,
                            "-L" + os.path.join(cuda_home, "lib64"), "-lcudart", "-lpthread"], capture_output=True, text=True)
    assert build.returncode == 0, build.stderr
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    run = subprocess.run([exe, "2"], capture_output=True, text=True, timeout=180, env=env)
    assert run.returncode == 0, run.stdout + run.stderr
    assert any(line.startswith("ok: 2 ranks") for line in run.stdout.splitlines()), run.stdout   # (NCCL may print its version first)
