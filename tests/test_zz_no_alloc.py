"""The allocation-free row sum (es_b200_rowsum_f32_noalloc) against the regular
entry point.

Some users of this library cannot allocate device memory at launch time: a
memgraph engine that has already claimed the whole GPU for its one big buffer,
or an event loop that cannot afford the device-wide stall of cudaMalloc.  For
them the library keeps the reduction's scratch in a fixed internal array.  This
test calls that entry point through the C ABI twice in a row (different data, so
stale scratch contents would show) and compares with the workspace-based kernel
of es_b200_launch_einsummable at the tolerance used for f32 sums elsewhere."""
import numpy as np
import pytest
import torch

import einsummable_b200 as es
from einsummable_b200 import _lib, einsummable_t, scalarop_t

pytestmark = pytest.mark.gpu


def regular_rowsum(km, x, rows, cols):
    e = einsummable_t([rows, cols], [[0, 1]], 1, scalarop_t.make_identity("f32"), "add")
    ws = km.build(e)
    out = torch.empty(rows, dtype=torch.float32, device="cuda:0")
    w = torch.empty(max(ws, 16), dtype=torch.uint8, device="cuda:0")
    km(e, None, out, [x], (w, ws) if ws else None)
    torch.cuda.synchronize()
    return out.cpu().numpy(), km.kernel_info(e)


# beyond the three basic shapes: more rows than one block of the second pass handles (1000), the
# largest row count the scratch allows (65536: one partial per row), and -- `offset` -- an input that
# starts one float past a 16-byte boundary although cols % 4 == 0, which takes the scalar loads
@pytest.mark.parametrize("rows,cols,offset", [(3, 1 << 20, 0), (64, 40000, 0), (5, 100003, 0), (1000, 4096, 0),
                                              (65536, 8, 0), (5, 4096, 1)])
def test_noalloc_rowsum_matches_regular_entry_point_twice(rows, cols, offset):
    km = es.kernel_manager_t(0)
    rng = np.random.default_rng(11)
    warm = torch.zeros(8, dtype=torch.float32, device="cuda:0")
    km.rowsum_f32_noalloc(None, warm[:2], warm, 2, 4)      # the first call on the device looks up the array
    torch.cuda.synchronize()
    for call in range(2):
        host = rng.standard_normal(rows * cols).astype(np.float32) * (call + 1)
        x = torch.from_numpy(np.concatenate([np.zeros(offset, np.float32), host])).cuda()[offset:]
        want, info = regular_rowsum(km, x.clone(), rows, cols)
        got = torch.full((rows,), float("nan"), dtype=torch.float32, device="cuda:0")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(0)[0]
        km.rowsum_f32_noalloc(None, got, x, rows, cols)
        torch.cuda.synchronize()
        # the point of the entry point: the device's free memory is what it was (nothing was allocated)
        assert torch.cuda.mem_get_info(0)[0] == free_before
        got = got.cpu().numpy()
        # f32 sums of N(0, s) terms: 1e-5 of the scale of the partial sums
        tol = 1e-5 * np.sqrt(cols) * (call + 1) * 4
        assert np.abs(got - want).max() <= tol, (call, info)
        exact = host.reshape(rows, cols).astype(np.float64).sum(axis=1)
        assert np.abs(got - exact).max() <= tol
    km.close()


def test_noalloc_rejects_sizes_beyond_its_scratch():
    km = es.kernel_manager_t(0)
    x = torch.zeros(16, dtype=torch.float32, device="cuda:0")
    with pytest.raises(es.es_error) as ei:
        km.rowsum_f32_noalloc(None, x, x, 65537, 4)
    assert ei.value.status == _lib.ES_NOT_SUPPORTED and "scratch" in str(ei.value)
    with pytest.raises(es.es_error):
        km.rowsum_f32_noalloc(None, x, 0, 4, 4)
    km.close()
