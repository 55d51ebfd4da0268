"""The allocation-free strided-rulebook entry point, `spconvb_down_map_static`.

Some hosts of this library may not allocate device memory once they are running:
a perception stack whose memory map is frozen after start-up, or a callback in
which `cudaMalloc` is forbidden or would stall the whole device.  They cannot
hand `spconvb_down_map` its workspace, so the library carries a fixed scratch
area of its own for them.  The variant must give exactly the results of the
ordinary entry point (all outputs are integers: tolerance 0), also on a second
call that finds the scratch area still holding the first call's contents.

This file is collected last on purpose, so that a run that stops at the first
failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from lidar_ai_solution_b200 import scenes  # noqa: E402

pytestmark = pytest.mark.gpu


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _static_down_map(ops, cabi, coords, n_ptr, grid, table, ksize, stride, pad, cap_out, status):
    """Calls the new entry point through the C ABI; every buffer is made by the caller."""
    dev = coords.device
    kvol = int(np.prod(ksize))
    oc = torch.zeros((cap_out, 4), dtype=torch.int32, device=dev)
    n_out = torch.zeros(1, dtype=torch.int32, device=dev)
    m = torch.full((kvol, cap_out), -1, dtype=torch.int32, device=dev)
    slots = cabi.lib().spconvb_hash_slots(cap_out)
    otab = torch.empty(slots, dtype=torch.int64, device=dev)
    rc = cabi.lib().spconvb_down_map_static(
        coords.data_ptr(), n_ptr.data_ptr(), coords.shape[0], 0, cabi.i3(grid), 1, cabi.i3(ksize),
        cabi.i3(stride), cabi.i3(pad), cabi.i3((1, 1, 1)), table.data_ptr(), table.numel(),
        oc.data_ptr(), n_out.data_ptr(), cap_out, m.data_ptr(), otab.data_ptr(), slots, 0,
        status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return rc, oc, n_out, m, otab


def test_static_scratch_variant_matches_workspace_variant_twice():
    from lidar_ai_solution_b200 import cabi, ops
    ksize, stride, pad = (3, 3, 3), (2, 2, 2), (1, 1, 1)
    # two different frames in a row: the second call meets the first call's bitmap
    for seed, n, grid in ((0, 60000, (41, 1440, 1440)), (1, 20000, (41, 720, 720))):
        coords = _dev(scenes.make_coords(n, grid, seed))
        n_ptr, st = ops.device_count(n), ops.new_status()
        table = ops.hash_build(coords, n_ptr, grid, status=st)
        cap_out = 4 * n
        ref_oc, ref_n, ref_m, ref_tab, og = ops.down_map(coords, n_ptr, grid, table, ksize, stride,
                                                         pad, cap_out=cap_out, status=st)
        rc, oc, n_out, m, otab = _static_down_map(ops, cabi, coords, n_ptr, grid, table, ksize,
                                                  stride, pad, cap_out, st)
        torch.cuda.synchronize()
        assert rc == cabi.OK, cabi.lib().spconvb_error_string(rc)
        assert int(st.cpu()[0]) == 0
        k = int(ref_n.item())
        assert k > 0 and int(n_out.item()) == k
        assert torch.equal(oc[:k], ref_oc[:k])
        assert torch.equal(m[:, :k], ref_m[:, :k])
        # the output hash tables answer the same queries: the next stage's SubM map
        sub_ref = ops.subm_map(ref_oc, ref_n, og, ref_tab)
        sub_new = ops.subm_map(oc, n_out, og, otab)
        torch.cuda.synchronize()
        assert torch.equal(sub_new[:, :k], sub_ref[:, :k])


def test_static_scratch_variant_rejects_grids_beyond_its_limit():
    from lidar_ai_solution_b200 import cabi, ops
    grid = (41, 1440, 1440)      # stride 1 keeps 85 M output cells: far beyond the scratch area
    need = cabi.lib().spconvb_down_workspace_bytes(cabi.i3(grid), 1)
    assert need > cabi.STATIC_SCRATCH_BYTES
    coords = _dev(scenes.make_coords(1000, grid, 2))
    n_ptr, st = ops.device_count(1000), ops.new_status()
    table = ops.hash_build(coords, n_ptr, grid, status=st)
    rc, _, n_out, _, _ = _static_down_map(ops, cabi, coords, n_ptr, grid, table, (3, 3, 3),
                                          (1, 1, 1), (1, 1, 1), 27000, st)
    torch.cuda.synchronize()
    assert rc == cabi.E_SCRATCH_LIMIT
    assert b"scratch" in cabi.lib().spconvb_error_string(rc)
    assert int(n_out.item()) == 0            # nothing was launched
