"""The C-ABI library without a GPU: it loads, exports every symbol the header declares,
its structs have the layout the ctypes binding assumes, and argument validation that does
not need a device answers with the documented error codes.  No kernel is launched."""
import ctypes as C
import os
import re

from megaattention_b200 import _cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "megaattn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ma_[a-z_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    names = _declared_functions()
    assert {"ma_query_device", "ma_plan_create", "ma_launch", "ma_read_status",
            "ma_plan_destroy", "ma_strerror", "ma_fused_prefill_noalloc",
            "ma_residual_rmsnorm", "ma_rope_qk"} <= set(names)
    for n in names:
        assert getattr(_cabi.lib, n) is not None, n
    assert set(names) == set(_cabi.EXPORTS)


def test_struct_layouts_match_the_header():
    # sizes / offsets computed by hand from the header (8-byte alignment for uint64_t)
    assert C.sizeof(_cabi.LaunchArgs) == 20
    assert C.sizeof(_cabi.Status) == 16
    assert _cabi.PlanDesc.Q.offset == 56
    assert _cabi.PlanDesc.peer_ready_count.offset == 56 + 21 * 8
    assert _cabi.PlanDesc.page_table.offset == 56 + 21 * 8 + 3 * 64
    assert _cabi.PlanDesc.fa_order.offset == 56 + 21 * 8 + 3 * 64 + 24
    assert _cabi.PlanDesc.peer_csym.offset == 56 + 21 * 8 + 3 * 64 + 32
    assert _cabi.PlanDesc.audit.offset == 56 + 21 * 8 + 3 * 64 + 32 + 64
    assert C.sizeof(_cabi.PlanDesc) == 56 + 21 * 8 + 3 * 64 + 32 + 64 + 8
    assert _cabi.NoAllocArgs.seqlens_q.offset == 40
    assert C.sizeof(_cabi.NoAllocArgs) == 40 + 2 * 8 + 5 * 8 + 8
    assert _cabi.RmsNormArgs.num_row_tiles.offset == 64 and C.sizeof(_cabi.RmsNormArgs) == 80


def test_error_strings_and_null_arguments():
    for code in (0, -1, -2, -3, -4, -5):
        assert _cabi.strerror(code) not in ("", "unknown error")
    assert _cabi.strerror(-99) == "unknown error"
    plan = C.c_void_p()
    assert _cabi.lib.ma_plan_create(None, C.byref(plan)) == _cabi.MA_ERR_INVALID
    assert _cabi.lib.ma_launch(None, None, None) == _cabi.MA_ERR_INVALID
    assert _cabi.lib.ma_read_status(None, None, None) == _cabi.MA_ERR_INVALID
    assert _cabi.lib.ma_fused_prefill_noalloc(None, None) == _cabi.MA_ERR_INVALID
    _cabi.lib.ma_plan_destroy(None)          # a no-op, must not crash


def test_shape_validation_happens_before_any_device_call():
    d = _cabi.PlanDesc()
    d.D, d.tp_size, d.H_local, d.H_kv = 64, 1, 8, 1       # head_dim 64 is not supported
    plan = C.c_void_p()
    assert _cabi.lib.ma_plan_create(C.byref(d), C.byref(plan)) == _cabi.MA_ERR_INVALID
    d.D, d.tp_size = 128, 9                                # more ranks than MA_MAX_TP
    assert _cabi.lib.ma_plan_create(C.byref(d), C.byref(plan)) == _cabi.MA_ERR_INVALID
    d.tp_size, d.H_local, d.H_kv = 1, 8, 3                 # q heads not a multiple of kv heads
    assert _cabi.lib.ma_plan_create(C.byref(d), C.byref(plan)) == _cabi.MA_ERR_INVALID
    a = _cabi.NoAllocArgs()
    a.H_local, a.H_kv, a.hidden, a.super_group_n_tiles, a.num_batch = 8, 1, 100, 4, 1
    q = (C.c_int32 * 1)(128)
    a.seqlens_q = q
    a.Q = a.K = a.V = a.W_o = a.out = 256
    assert _cabi.lib.ma_fused_prefill_noalloc(C.byref(a), None) == _cabi.MA_ERR_INVALID
    a.hidden, a.num_batch = 128, 513
    assert _cabi.lib.ma_fused_prefill_noalloc(C.byref(a), None) == _cabi.MA_ERR_CAPACITY


def test_ctypes_mirror_agrees_with_the_compiled_header(tmp_path):
    """Compile the header with the C compiler and compare sizeof / offsetof of every field
    of every struct with the ctypes mirror (the hand-computed numbers above only pin a few)."""
    import shutil
    import subprocess
    cc = shutil.which("gcc") or shutil.which("cc")
    assert cc, "a C compiler is part of the build environment"
    pairs = {"ma_devinfo": _cabi.DevInfo, "ma_plan_desc": _cabi.PlanDesc,
             "ma_launch_args": _cabi.LaunchArgs, "ma_status": _cabi.Status,
             "ma_noalloc_args": _cabi.NoAllocArgs, "ma_rmsnorm_args": _cabi.RmsNormArgs,
             "ma_rope_args": _cabi.RopeArgs}
    lines = ['#include <stdio.h>', '#include <stddef.h>',
             '#include "%s"' % os.path.join(ROOT, "include", "megaattn_b200.h"),
             'int main(void) {']
    for cname, ct in pairs.items():
        lines.append('  printf("%s sizeof %%zu\\n", sizeof(%s));' % (cname, cname))
        for fname, *_ in ct._fields_:
            lines.append('  printf("%s %s %%zu\\n", offsetof(%s, %s));' % (cname, fname, cname, fname))
    lines += ['  return 0;', '}']
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run([cc, "-std=c99", "-o", str(exe), str(src)], check=True, capture_output=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    seen = 0
    for ln in out.splitlines():
        cname, fname, val = ln.split()
        ct = pairs[cname]
        want = C.sizeof(ct) if fname == "sizeof" else getattr(ct, fname).offset
        assert int(val) == want, (cname, fname, val, want)
        seen += 1
    assert seen == sum(len(ct._fields_) + 1 for ct in pairs.values())


def test_consumer_entry_point_validates_before_any_device_call():
    """ma_residual_rmsnorm: null, misaligned and over-wide arguments are refused on the host
    (this machine has no GPU: anything that reached CUDA would fail differently)."""
    ok = dict(csym=1 << 20, residual_in=2 << 20, weight=3 << 20, residual_out=2 << 20,
              normed_out=4 << 20, cu_q=5 << 20, fa_b=6 << 20, fa_mb=7 << 20,
              num_row_tiles=3, hidden=4096, row_pitch=4096, eps=1e-6)

    def call(**kw):
        a = _cabi.RmsNormArgs(**{**ok, **kw})
        return _cabi.lib.ma_residual_rmsnorm(C.byref(a), None)

    assert _cabi.lib.ma_residual_rmsnorm(None, None) == _cabi.MA_ERR_INVALID
    assert call(weight=0) == _cabi.MA_ERR_INVALID
    assert call(normed_out=(4 << 20) + 8) == _cabi.MA_ERR_INVALID          # 16-byte accesses
    assert call(hidden=4100) == _cabi.MA_ERR_INVALID                       # not a multiple of 8
    assert call(row_pitch=2048) == _cabi.MA_ERR_INVALID                    # narrower than hidden
    assert call(eps=-1.0) == _cabi.MA_ERR_INVALID
    assert call(hidden=16392, row_pitch=16392) == _cabi.MA_ERR_CAPACITY
    assert call(num_row_tiles=0) == _cabi.MA_OK                            # nothing to do


def test_rope_entry_point_validates_before_any_device_call():
    ok = dict(q=1 << 20, k=2 << 20, cu_q=3 << 20, cu_k=4 << 20, token_batch=5 << 20,
              inv_freq=6 << 20, tot_q=10, H_local=8, H_kv=1, reserved0=0)

    def call(**kw):
        a = _cabi.RopeArgs(**{**ok, **kw})
        return _cabi.lib.ma_rope_qk(C.byref(a), None)

    assert _cabi.lib.ma_rope_qk(None, None) == _cabi.MA_ERR_INVALID
    assert call(inv_freq=0) == _cabi.MA_ERR_INVALID
    assert call(q=(1 << 20) + 2) == _cabi.MA_ERR_INVALID                   # 16-byte accesses
    assert call(H_kv=0) == _cabi.MA_ERR_INVALID
    assert call(tot_q=-1) == _cabi.MA_ERR_INVALID
    assert call(tot_q=0) == _cabi.MA_OK                                    # nothing to do
