"""Index tables that address rows outside their tensor: the kernels skip the access, raise the status word (which the
host turns into an exception) and leave everything outside the output tensor untouched (canary rows)."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "helpers"))

pytestmark = pytest.mark.gpu


def _status_raises(match="outside its tensor"):
    from lmms_engine_b200.ops import _cuda

    with pytest.raises(RuntimeError, match=match):
        _cuda.check_status()
    _cuda.check_status()  # cleared by the report


@pytest.mark.parametrize("n_src,n_out,H", [(5, 7, 64), (128, 129, 256), (1, 1, 8)])
def test_gather_and_scatter_rows_skip_indices_past_the_end(n_src, n_out, H):
    from canary import Canary

    from lmms_engine_b200.ops import _cuda

    torch.manual_seed(0)
    src = torch.randn(n_src, H, device="cuda", dtype=torch.bfloat16)
    idx = torch.randint(0, n_src, (n_out,), device="cuda")
    idx[0] = -1  # "no row": zeros
    bad = idx.clone()
    bad[-1] = n_src + 3  # past the end
    out = Canary(n_out, H)
    st = _cuda.status_word(src.device)
    _cuda.call("b200_gather_rows", src.data_ptr(), bad.data_ptr(), out.t.data_ptr(), n_out, H, n_src, st.data_ptr(), _cuda.stream())
    want = src.index_select(0, idx.clamp(min=0))
    want[0] = 0
    assert torch.equal(out.t[:-1], want[:-1]) and float(out.t[-1].abs().sum()) == 0.0  # the bad row reads as zeros
    out.check("gather_rows")
    _status_raises()
    # in-range tables raise nothing
    _cuda.call("b200_gather_rows", src.data_ptr(), idx.data_ptr(), out.t.data_ptr(), n_out, H, n_src, st.data_ptr(), _cuda.stream())
    _cuda.check_status()
    assert torch.equal(out.t, want)
    # scatter: the row aimed past the end is dropped
    dst = Canary(n_src, H, fill=torch.zeros(n_src, H))
    perm = torch.randperm(n_src, device="cuda")
    rows = torch.randn(n_src, H, device="cuda", dtype=torch.bfloat16)
    bad_perm = perm.clone()
    bad_perm[0] = n_src  # one past the end
    _cuda.call("b200_scatter_rows", rows.data_ptr(), bad_perm.data_ptr(), dst.t.data_ptr(), n_src, H, 0, n_src, st.data_ptr(), _cuda.stream())
    dst.check("scatter_rows")
    _status_raises()
    assert torch.equal(dst.t[perm[1:]], rows[1:]) and float(dst.t[perm[0]].abs().sum()) == 0.0


def test_moe_combine_skips_routing_entries_past_the_end():
    from canary import Canary

    from lmms_engine_b200.ops import _cuda
    from lmms_engine_b200.ops import moe as moe_ops  # noqa: F401  (registers the launchers)

    torch.manual_seed(0)
    T, k, H, rows = 9, 2, 64, 24
    src = torch.randn(rows, H, device="cuda", dtype=torch.bfloat16)
    row_of = torch.randint(0, rows, (T, k), device="cuda", dtype=torch.int32)
    w = torch.rand(T, k, device="cuda")
    bad = row_of.clone()
    bad[3, 1] = rows + 100
    out = Canary(T, H)
    st = _cuda.status_word(src.device)
    _cuda.call("b200_moe_combine", src.data_ptr(), bad.data_ptr(), w.data_ptr(), out.t.data_ptr(), T, k, H, rows, st.data_ptr(), _cuda.stream())
    out.check("moe_combine")
    _status_raises()
    keep = torch.ones(T, k, device="cuda")
    keep[3, 1] = 0
    want = ((w * keep)[..., None] * src.float()[row_of.long()]).sum(1)
    assert (out.t.float() - want).abs().max() < 0.05
    dw = torch.full((T, k), 7.0, device="cuda")
    dout = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    _cuda.call("b200_moe_combine_bwd_w", dout.data_ptr(), src.data_ptr(), bad.data_ptr(), dw.data_ptr(), T * k, k, H, rows, st.data_ptr(), _cuda.stream())
    _status_raises()
    assert float(dw[3, 1]) == 0.0
    ref = (dout.float()[:, None] * src.float()[row_of.long()]).sum(-1)
    mask = keep.bool()
    assert (dw[mask] - ref[mask]).abs().max() < 0.5


def test_debug_build_is_selected_by_the_environment():
    """The debug libraries live beside the release ones and are chosen at import time; this process runs the release build."""
    from lmms_engine_b200 import _native
    from lmms_engine_b200.ops import _cuda
    from lmms_engine_b200.ops import moe as moe_ops  # noqa: F401

    assert _native.DEBUG_BOUNDS == (os.environ.get("LMMS_B200_DEBUG_BOUNDS", "0") == "1")
    assert _native.LIBDIR.name == ("_lib_dbg" if _native.DEBUG_BOUNDS else "_lib")
    assert _cuda.fn("b200_moe_debug_bad_index")() == (0 if _native.DEBUG_BOUNDS else -1)
