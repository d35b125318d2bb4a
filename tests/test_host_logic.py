"""Host-side logic that needs no GPU: the C-ABI library's exports, argument
validation before the driver is touched, the slab allocator, the kernel
"compiler" front end and the dispatcher's launch lists (against a fake runtime).
Mirrors the reference's own no-GPU tests (tests/test_hip_bridge.py,
tests/test_hardware_safety.py, tests/test_slab_allocator.py, tests/test_codegen.py)."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

from vte_b200.bridge.cuda_runtime import CudaRuntime, EXPORTED_SYMBOLS, FastPlan, load_library
from vte_b200.bridge.errors import CudaRuntimeError, CudaSafetyError, HIPSafetyError, MemoryGuardianOOMError
from vte_b200.bridge.memory import MemoryRegion, SlabAllocator
from vte_b200.compiler.codegen import CodegenEngine, _sanitize_var
from vte_b200.compiler.signatures import KERNEL_SIGNATURES
from vte_b200.core.split_kv_attention import SplitKVAttentionDispatcher, choose_split_count

ROOT = Path(__file__).resolve().parent.parent


# ----------------------------------------------------------------------------- library
def test_library_exports_every_declared_symbol(built_library):
    header = (ROOT / "include" / "vteb200.h").read_text()
    declared = set(re.findall(r"\b(vteb_[a-z0-9_]+)\s*\(", header))
    assert len(declared) > 40
    lib = ctypes.CDLL(str(built_library))
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in include/vteb200.h but not exported"
    load_library(str(built_library))
    assert declared == set(EXPORTED_SYMBOLS), declared ^ set(EXPORTED_SYMBOLS)


def test_library_refuses_work_before_init(built_library):
    lib = load_library(str(built_library))
    p = ctypes.c_void_p()
    assert lib.vteb_malloc(ctypes.byref(p), 16) == -2           # VTEB_ERR_NOT_INITIALIZED
    assert b"vteb_init" in lib.vteb_last_error_string()
    assert lib.vteb_device_synchronize() == -2


def test_plan_is_pure_host_arithmetic(built_library):
    lib = load_library(str(built_library))
    for hq, hkv, d, hg, nhg in [(12, 2, 128, 2, 1), (32, 8, 64, 8, 1), (8, 2, 256, 1, 2), (32, 8, 128, 4, 2),
                                (16, 16, 64, 8, 2), (4, 1, 64, 1, 1)]:
        plan = FastPlan()
        assert lib.vteb_split_kv_plan(hq, hkv, d, ctypes.byref(plan)) == 0
        assert plan.ok == 1 and plan.hg == hg and plan.n_hgroups == nhg
        assert plan.smem_bytes <= 227 * 1024 and plan.nstages >= 2 and plan.tile % 16 == 0
        assert plan.threads == 320 and plan.combine_dsplit == d // 32
        small = FastPlan()
        assert lib.vteb_split_kv_plan_compact(hq, hkv, d, ctypes.byref(small)) == 0
        if small.ok:
            assert small.threads == 256 and small.hg <= 6 and small.smem_bytes <= 227 * 1024 and small.nstages >= 2
            assert small.hg * (2 if d == 256 else 1) <= 6
    for hq, hkv, d in [(32, 2, 128), (12, 2, 96), (12, 5, 128), (12, 0, 128)]:   # group 16, odd dim, non-divisor
        plan = FastPlan()
        assert lib.vteb_split_kv_plan(hq, hkv, d, ctypes.byref(plan)) == 0
        assert plan.ok == 0


def test_runtime_without_device_fails_loudly(built_library):
    rt = CudaRuntime(str(built_library))
    with pytest.raises(CudaSafetyError):
        rt.safe_malloc(16, "x")                                  # not initialised
    try:
        rt.initialize()
    except CudaRuntimeError:
        return                                                   # no GPU here: the only acceptable outcome
    rt.cleanup()                                                 # a GPU box: initialisation is allowed to work


def test_missing_library_is_an_error():
    with pytest.raises(CudaRuntimeError):
        load_library("/nonexistent/libvteb200.so")


# ----------------------------------------------------------------------------- fake runtime
class FakeRuntime:
    """Stands in for CudaRuntime the way tests/test_slab_allocator.py backs the
    slab with host memory: addresses are fake, nothing is dereferenced."""
    def __init__(self, sms=148):
        self.sms = sms
        self.loaded = []
        self.allocs = {}
        self._next = 0x7000_0000_0000
        self._lib = load_library()

    def get_num_cus(self): return self.sms
    def get_gpu_architecture(self): return "sm_100a"
    def combine_rows_epl(self, rows, d): return self._lib.vteb_combine_rows_epl(rows, d)
    def split_kv_plan(self, hq, hkv, d, compact=False):
        plan = FastPlan()
        (self._lib.vteb_split_kv_plan_compact if compact else self._lib.vteb_split_kv_plan)(hq, hkv, d, ctypes.byref(plan))
        return plan
    def safe_malloc(self, n, tag="x"):
        p = self._next
        self._next += (n + 255) // 256 * 256
        self.allocs[p] = n
        return ctypes.c_void_p(p)
    def safe_free(self, p, tag="x"):
        del self.allocs[p.value]
        return True
    def safe_memset(self, p, n, tag="x", value=0): return True
    def load_kernel(self, path, name):
        self.loaded.append((Path(path).name, name))
        return ctypes.c_void_p(1), ctypes.c_void_p(0x1000 + len(self.loaded))


class FakeCodegen:
    def __init__(self): self.calls = []
    def load_kernel_safe(self, hip, template, arch, symbol, **kw):
        self.calls.append((template, arch, symbol, kw))
        return hip.load_kernel(f"{template}.cubin", symbol)


def make_dispatcher(meta=None, **kw):
    rt = FakeRuntime()
    alloc = SlabAllocator(rt, 180 << 30, requested_pool_size=1 << 30)
    alloc.initialize()
    meta = meta or {'attention.head_count': 12, 'attention.head_count_kv': 2, 'attention.key_length': 128}
    cg = FakeCodegen()
    return SplitKVAttentionDispatcher(rt, cg, meta, allocator=alloc, **kw), rt, cg, alloc


def mapping(layer=0, stride=32768 * 2 * 128):
    base = 0x7100_0000_0000
    return {f'blk.{layer}.q_proj.output': base, f'blk.{layer}.k_proj.output': base + 0x10000,
            f'blk.{layer}.v_proj.output': base + 0x20000, f'blk.{layer}.attention.output': base + 0x30000,
            f'blk.{layer}.kv_cache.k': base + 0x100000, f'blk.{layer}.kv_cache.v': base + 0x4000000,
            'kv_batch_stride_elements': stride}


# ----------------------------------------------------------------------------- dispatcher
def test_fast_launch_list_shapes_and_signatures():
    d, rt, cg, _ = make_dispatcher(context_length=32768, batch_size=1, fused_combine=False, variant="full")
    assert d.enabled and not d.compat and d.max_chunks == 148 and not d.compact
    launches = d.build_launches(0, mapping(), 0x7200_0000_0000, batch=1)
    assert len(launches) == 3
    (fa, aa, ga, ba, sa), (fp, ap, gp, bp, sp), (fr, ar, gr, br, sr) = launches
    assert ga == (1, 2, 1) and ba == (128, 1, 1) and sa == 0 and len(aa) == len(KERNEL_SIGNATURES["kv_cache_append_kernel"])
    assert gp == (148, 1, 1) and bp == (320, 1, 1) and 100_000 < sp <= 227 * 1024
    assert len(ap) == len(KERNEL_SIGNATURES["vteb_split_kv_partial_d128_kernel"])
    assert gr == (12 * 4, 1, 1) and br == (256, 1, 1) and sr == 148 * 4
    assert len(ar) == len(KERNEL_SIGNATURES["vteb_split_kv_combine_f16_kernel"])
    # the first 13 arguments of the split launch are the reference kernel's, in its order
    for arg, typ in zip(ap, KERNEL_SIGNATURES["flash_attention_split_kv_partial_kernel"]):
        assert isinstance(arg, typ)
    assert ap[6].value == 12 and ap[7].value == 2 and ap[8].value == 128 and ap[12].value == 148
    assert abs(ap[9].value - 1 / np.sqrt(128)) < 1e-7
    symbols = [s for _, s in rt.loaded]
    assert symbols == ["kv_cache_append_kernel", "vteb_split_kv_partial_d128_kernel", "vteb_split_kv_combine_f16_kernel"]
    # scratch: one set for all layers, sized as the reference sizes it
    pm, pl, po = d.partial_buffers
    assert pm.size == 12 * 148 * 4 and po.size == 12 * 148 * 128 * 4
    again = d.build_launches(1, mapping(1), 0x7200_0000_0000, batch=1)
    assert again[1][1][3].value == ap[3].value


def test_fused_launch_list_is_append_plus_one_launch():
    d, rt, cg, _ = make_dispatcher(context_length=32768, batch_size=1, output_f32=True, fused_combine=True)
    assert d.fused_combine
    launches = d.build_launches(0, mapping(), 0x7200_0000_0000, batch=1)
    assert len(launches) == 2
    fp, ap, gp, bp, sp = launches[1]
    assert len(ap) == len(KERNEL_SIGNATURES["vteb_split_kv_partial_d128_kernel"])
    assert ap[22].value == 2 and ap[21].value == mapping()['blk.0.attention.output']
    assert all(isinstance(a, ctypes.Structure) and ctypes.sizeof(a) == 128 for a in ap[23:25])   # the two tensor maps
    # three KV heads per group cannot use all eight consumer warps: no in-launch combine
    d2, *_ = make_dispatcher({'attention.head_count': 12, 'attention.head_count_kv': 3, 'attention.key_length': 128},
                             fused_combine=True)
    assert not d2.fused_combine and len(d2.build_launches(0, mapping(), 0x7200_0000_0000)) == 3


def test_fused_rope_launch_list_and_standalone_rotation_launch():
    meta = {'attention.head_count': 8, 'attention.head_count_kv': 2, 'attention.key_length': 256,
            'rope_type': 2, 'rotary_dim': 64}
    d, rt, cg, _ = make_dispatcher(meta, context_length=4096, batch_size=4, fuse_rope=True)
    m = mapping()
    with pytest.raises(CudaSafetyError):
        d.build_launches(0, m, 0x7200_0000_0000, batch=4)              # no tables in the mapping
    m['rope_cos'], m['rope_sin'] = 0x7300_0000_0000, 0x7300_1000_0000
    launches = d.build_launches(0, m, 0x7200_0000_0000, batch=4)
    symbols = [s for _, s in rt.loaded]
    assert symbols[:2] == ["kv_cache_append_rope_kernel", "vteb_split_kv_partial_rope_d256_kernel"]
    (fa, aa, ga, ba, sa), (fp, ap, gp, bp, sp) = launches[:2]
    assert len(aa) == len(KERNEL_SIGNATURES["kv_cache_append_rope_kernel"]) == 12
    assert len(ap) == len(KERNEL_SIGNATURES["vteb_split_kv_partial_rope_d256_kernel"]) == 31
    assert [a.value for a in aa[-4:]] == [0x7300_0000_0000, 0x7300_1000_0000, 2, 64]
    assert [a.value for a in ap[-6:-2]] == [0x7300_0000_0000, 0x7300_1000_0000, 2, 64]
    assert [a.value for a in ap[-2:]] in ([0, 0], [None, None])           # no fused append asked for
    assert ga == (4, 2, 1) and ba == (256, 1, 1)
    # the standalone launch: the reference's eleven arguments and its grid rule
    fn, args, grid, block, smem = d.build_rope_launch(m, 0x7200_0000_0000, batch=4)
    assert rt.loaded[-1][1] == "rope_kernel" and len(args) == len(KERNEL_SIGNATURES["rope_kernel"]) == 11
    assert grid == (8 * 256 // 256, 4, 1) and block == (256, 1, 1) and smem == 0
    assert [a.value for a in args[4:8]] == [1, 8, 2, 256] and [a.value for a in args[9:]] == [2, 64]
    # options the rotation cannot be combined with, and widths the kernel has no code for
    meta128 = {'attention.head_count': 12, 'attention.head_count_kv': 2, 'attention.key_length': 128}
    with pytest.raises(CudaSafetyError):
        make_dispatcher(meta128, fuse_rope=True, compat=True)
    dc, rtc, *_ = make_dispatcher(meta128, fuse_rope=True, context_length=4096)           # one sequence: compact shape
    m128 = dict(mapping(), rope_cos=0x7300_0000_0000, rope_sin=0x7300_1000_0000)
    assert dc.compact and len(dc.build_launches(0, m128, 0x7200_0000_0000)[1][1]) == 31
    assert rtc.loaded[1][1] == "vteb_split_kv_partial_compact_rope_d128_kernel"
    # fused append: no append launch; the split launch carries the new rows; without rotation the type is -1
    df, rtf, *_ = make_dispatcher(meta128, fuse_append=True, context_length=4096)
    lf = df.build_launches(0, mapping(), 0x7200_0000_0000)
    assert len(lf) == 2 and rtf.loaded[1][1] == "vteb_split_kv_partial_compact_rope_d128_kernel"
    tail = [a.value for a in lf[0][1][-6:]]
    assert tail[2:4] == [-1, 0] and tail[4:] == [mapping()['blk.0.k_proj.output'], mapping()['blk.0.v_proj.output']]
    dfr, *_ = make_dispatcher(meta128, fuse_append=True, fuse_rope=True, context_length=4096)
    tail = [a.value for a in dfr.build_launches(0, m128, 0x7200_0000_0000)[0][1][-6:]]
    assert tail[:4] == [0x7300_0000_0000, 0x7300_1000_0000, 0, 128] and tail[4] == mapping()['blk.0.k_proj.output']
    with pytest.raises(CudaSafetyError):
        make_dispatcher(meta128, fuse_append=True, compat=True)
    # the split kernel copies the new rows 16 bytes at a time: an 8-byte-aligned projection is refused
    for name in ('blk.0.k_proj.output', 'blk.0.v_proj.output'):
        skew = dict(mapping())
        skew[name] += 8
        with pytest.raises(CudaSafetyError, match="16-byte aligned"):
            df.build_launches(0, skew, 0x7200_0000_0000)
    with pytest.raises(CudaSafetyError):
        make_dispatcher(dict(meta, rotary_dim=48), fuse_rope=True)
    with pytest.raises(CudaSafetyError):
        make_dispatcher(dict(meta, rope_type=3), fuse_rope=True)


def test_rope_cache_builder_matches_the_pinned_tables():
    from oracle import attention_oracle as orc
    from vte_b200.workloads import build_rope_cache
    for width, theta in ((128, 1e6), (64, 1e7), (256, 1e4)):
        cos, sin = build_rope_cache(300, width, theta)
        oc, os_ = orc.rope_tables(300, width, theta)
        assert cos.dtype == np.float16 and cos.shape == (300, width)
        assert np.array_equal(cos, oc) and np.array_equal(sin, os_)
        assert np.array_equal(cos[:, :width // 2], cos[:, width // 2:])


def test_tensor_maps_are_passed_when_the_cache_is_a_matrix_of_rows():
    from vte_b200.bridge.cuda_runtime import KvTensorMap
    from vte_b200.core.split_kv_attention import FLAG_TENSOR_MAPS

    class MapRuntime(FakeRuntime):
        def __init__(self):
            super().__init__()
            self.encoded = []
        def kv_tensor_map(self, ptr, n_rows, row_halves, box_rows):
            self.encoded.append((ptr, n_rows, row_halves, box_rows))
            tm = KvTensorMap()
            tm.opaque[0] = ptr
            return tm

    rt = MapRuntime()
    alloc = SlabAllocator(rt, 180 << 30, requested_pool_size=1 << 30)
    alloc.initialize()
    meta = {'attention.head_count': 12, 'attention.head_count_kv': 2, 'attention.key_length': 128}
    d = SplitKVAttentionDispatcher(rt, FakeCodegen(), meta, allocator=alloc, context_length=32768, batch_size=1)
    m = mapping()
    ap = d.build_launches(0, m, 0x7200_0000_0000, batch=1)[1][1]
    assert ap[15].value & FLAG_TENSOR_MAPS
    assert ap[23].opaque[0] == m['blk.0.kv_cache.k'] and ap[24].opaque[0] == m['blk.0.kv_cache.v']
    # rows = stride / (Hkv * D), boxes of `tile` rows; encoded once per cache, reused on the next capture
    assert rt.encoded == [(m['blk.0.kv_cache.k'], 32768, 256, d._plan.tile), (m['blk.0.kv_cache.v'], 32768, 256, d._plan.tile)]
    d.build_launches(0, m, 0x7200_0000_0000, batch=1)
    assert len(rt.encoded) == 2
    # a sequence stride that is not a whole number of position rows: 16-byte copies only
    odd = dict(m, kv_batch_stride_elements=32768 * 256 + 8)
    ap2 = d.build_launches(0, odd, 0x7200_0000_0000, batch=1)[1][1]
    assert not (ap2[15].value & FLAG_TENSOR_MAPS) and ap2[23].opaque[0] == 0
    # switched off by the caller
    d2 = SplitKVAttentionDispatcher(rt, FakeCodegen(), meta, allocator=alloc, context_length=32768, batch_size=1,
                                    tensor_maps=False)
    assert not (d2.build_launches(0, m, 0x7200_0000_0000, batch=1)[1][1][15].value & FLAG_TENSOR_MAPS)


def test_kv_range_combine_launch_is_rewritten_for_the_fused_exchange():
    from vte_b200.core.kv_shard import KVRangeShardedDecode, PairBoards
    sh = object.__new__(KVRangeShardedDecode)
    sh.world, sh.rank, sh.L, sh.rows, sh.fused_merge = 4, 2, 28, 12, True
    sh._pair_boards, sh._step_ptr, sh._combine_push_fn = PairBoards(), 0x7400_0000_0040, ctypes.c_void_p(0x99)
    sh._board = ctypes.c_void_p(0x7400_0000_0000)
    class Ex: D = 128
    class Disp: work_ptr = 0x7500_0000_0000
    class Merged: ptr = 0x7600_0000_0000
    Ex.dispatcher = Disp; sh.ex = Ex; sh.merged = Merged
    vp, ci = ctypes.c_void_p, ctypes.c_int
    combine = ("combine_fn", [vp(1), vp(2), vp(3), vp(4), ci(12), ci(128), ci(148), ci(4), vp(5)], (48, 1, 1), (256, 1, 1), 592)
    out = sh._fuse_push_into_combine(3, ["append", "split", combine])
    assert out[:2] == ["append", "split"]
    fn, args, grid, block, smem = out[2]
    assert fn is sh._combine_push_fn and (grid, block, smem) == ((48, 1, 1), (256, 1, 1), 592)
    sig = KERNEL_SIGNATURES["vteb_split_kv_combine_push_kernel"]
    assert len(args) == len(sig) == 19 and all(isinstance(a, t) for a, t in zip(args, sig))
    assert [a.value for a in args[10:15]] == [4, 2, 3, 28, 12]
    assert args[17].value == Merged.ptr + 3 * 12 * 128 * 4 and args[18].value == Disp.work_ptr + 4
    sh.fused_merge = False
    assert sh._fuse_push_into_combine(3, [combine])[0][1][17].value in (0, None)


def test_compact_shape_selection():
    d, rt, cg, _ = make_dispatcher(context_length=32768, batch_size=1, variant="compact")
    assert d.compact and d.max_chunks == 148
    fp, ap, gp, bp, sp = d.build_launches(0, mapping(), 0x7200_0000_0000, batch=1)[1]
    assert gp == (148, 1, 1) and bp == (256, 1, 1) and 100_000 < sp <= 227 * 1024
    assert [s for _, s in rt.loaded][1] == "vteb_split_kv_partial_compact_d128_kernel"
    # auto: compact for one sequence, full for a batch
    assert make_dispatcher(context_length=32768, batch_size=1, variant="auto")[0].compact
    assert not make_dispatcher(context_length=32768, batch_size=4, variant="auto")[0].compact
    assert not make_dispatcher(context_length=1 << 20, batch_size=1)[0].compact          # auto is the default
    # 256-wide heads have a compact kernel too (one KV head x two column halves x three block streams)
    wide = make_dispatcher({'attention.head_count': 8, 'attention.head_count_kv': 2, 'attention.key_length': 256},
                           variant="compact")[0]
    assert wide.compact
    # eight 64-wide KV heads: four per item in the compact shape (six consumer warps), eight in the full one
    many = make_dispatcher({'attention.head_count': 32, 'attention.head_count_kv': 8, 'attention.key_length': 64},
                           variant="compact")[0]
    assert many.compact and many._plan.hg == 4 and many._plan.n_hgroups == 2
    with pytest.raises(CudaSafetyError):
        make_dispatcher(variant="lite")


def test_compat_launch_list_is_the_reference_geometry():
    d, rt, cg, _ = make_dispatcher(context_length=4096, batch_size=1, fixed_chunk_size="auto", compat=True)
    assert d.chunk_size == 8 and d.max_chunks == 512               # 148 "CUs" -> clamp(round(1024/148), 8, 64) = 8
    launches = d.build_launches(0, mapping(), 0x7200_0000_0000)
    assert [(g, b, s) for _, _, g, b, s in launches] == [((1, 2, 1), (128, 1, 1), 0), ((1, 12, 512), (128, 1, 1), 1024),
                                                         ((1, 12, 1), (128, 1, 1), 2048)]
    assert [len(a) for _, a, _, _, _ in launches] == [8, 13, 7]
    assert all(kw == {'split_kv_chunk_size': 8} for _, _, _, kw in cg.calls)
    assert [s for _, s in rt.loaded] == ["kv_cache_append_kernel", "flash_attention_split_kv_partial_kernel",
                                         "flash_attention_split_kv_reduce_kernel"]


def test_dispatcher_switches_and_fallbacks(monkeypatch):
    d, *_ = make_dispatcher({'attention.head_count': 32, 'attention.head_count_kv': 2, 'attention.key_length': 128})
    assert d.compat                                               # group 16 is outside the fast kernel
    monkeypatch.setenv("VTE_DISABLE_ATTN_SPLITKV", "1")
    d2, *_ = make_dispatcher()
    assert not d2.enabled
    monkeypatch.delenv("VTE_DISABLE_ATTN_SPLITKV")
    rt = FakeRuntime()
    assert not SplitKVAttentionDispatcher(rt, FakeCodegen(), {}, allocator=None).enabled
    d3, *_ = make_dispatcher({'attention.head_count': 12, 'attention.head_count_kv': 2, 'attention.key_length': 128,
                              'attention_scale': 0.015625})
    assert d3.build_launches(0, mapping(), 0x7200_0000_0000)[1][1][9].value == 0.015625


def test_dispatcher_rejects_bad_arguments_before_any_launch():
    d, *_ = make_dispatcher(context_length=4096, batch_size=2)
    good = mapping(stride=4096 * 2 * 128)
    with pytest.raises(CudaSafetyError):
        d.build_launches(0, good, 0)                               # null offsets
    with pytest.raises(CudaSafetyError):
        d.build_launches(0, good, 0x7200_0000_0000, batch=3)       # above batch_size
    bad = dict(good); bad['blk.0.kv_cache.k'] += 2
    with pytest.raises(CudaSafetyError):
        d.build_launches(0, bad, 0x7200_0000_0000)                 # misaligned cache
    bad = dict(good); bad['kv_batch_stride_elements'] = 2 ** 31
    with pytest.raises(CudaSafetyError):
        d.build_launches(0, bad, 0x7200_0000_0000)
    bad = dict(good); del bad['blk.0.attention.output']
    with pytest.raises(CudaSafetyError):
        d.build_launches(0, bad, 0x7200_0000_0000)
    bad = dict(good); bad['kv_batch_stride_elements'] = 0
    with pytest.raises(CudaSafetyError):
        d.build_launches(0, bad, 0x7200_0000_0000, batch=2)
    assert issubclass(CudaSafetyError, Exception) and HIPSafetyError is CudaSafetyError


def test_kv_cache_name_fallbacks():
    d, *_ = make_dispatcher(context_length=2048, batch_size=1)
    m = mapping(stride=2048 * 2 * 128)
    k, v = m.pop('blk.0.kv_cache.k'), m.pop('blk.0.kv_cache.v')
    m['kv_cache.layer_0.k'], m['kv_cache.layer_0.v'] = k, v
    assert d._resolve_kv_cache_ptrs(0, m) == (k, v)
    del m['kv_cache.layer_0.k'], m['kv_cache.layer_0.v']
    m['KV Cache Pool'] = 0x7300_0000_0000
    half = 1 * 2 * 128 * 2 * 2048
    assert d._resolve_kv_cache_ptrs(3, m) == (0x7300_0000_0000 + 3 * 2 * half, 0x7300_0000_0000 + 3 * 2 * half + half)


def test_split_count_policy():
    assert choose_split_count(148, 1, 1, 32768) == 148            # one sequence: one wave
    assert choose_split_count(148, 1, 2, 32768) == 74
    assert choose_split_count(148, 64, 1, 16384) == 16            # ragged batch: ~4 items per SM -> 1024-position chunks
    assert choose_split_count(148, 16, 1, 65536) == 64
    assert choose_split_count(148, 4, 1, 4096) == 8               # small batch: 512-position chunks, the smallest aimed at
    assert choose_split_count(148, 2, 1, 100) == 1


# ----------------------------------------------------------------------------- allocator
def test_slab_allocator_alignment_reuse_and_overlap():
    rt = FakeRuntime()
    a = SlabAllocator(rt, 100 << 20, requested_pool_size=1 << 20)
    a.initialize()
    assert a.total_size == 1 << 20
    x = a.allocate(100, "x", MemoryRegion.SCRATCH)
    y = a.allocate(300, "y", MemoryRegion.KV_CACHE)
    z = a.allocate(64, "z", MemoryRegion.ACTIVATIONS)
    assert x.ptr % 128 == 0 and y.ptr == x.ptr + 128 and z.ptr == y.ptr + 384
    assert a.validate_pointer(y.ptr + 8, 200) and not a.validate_pointer(y.ptr + 8, 400)
    assert not a.validate_pointer(a.slab_base - 1, 1)
    a.free(y)
    assert not a.validate_pointer(y.ptr, 1)
    w = a.allocate(256, "w", MemoryRegion.SCRATCH)                # best fit: the hole y left
    assert w.ptr == y.ptr
    with pytest.raises(CudaSafetyError):
        a.free(y)                                                 # double free
    with pytest.raises(CudaSafetyError):
        a.allocate(0, "zero", MemoryRegion.SCRATCH)
    with pytest.raises(CudaSafetyError):
        a.allocate(2 << 20, "huge", MemoryRegion.SCRATCH)
    a.free(z)                  # merges with the 128 B left of y's hole; the merged tail returns to the bump pointer
    assert a.get_stats()["holes"] == 0 and a.current_offset == 384
    stats = a.get_stats()                                         # the reference's keys (vte/bridge/memory.py:185-193)
    assert stats["total_bytes"] == 1 << 20 and stats["used_bytes"] == 384 and stats["active_blocks"] == 2
    assert stats["free_bytes"] == (1 << 20) - 384
    with pytest.raises(CudaSafetyError):
        a.initialize()                                            # a second initialize raises, as the reference's does
    big = SlabAllocator(rt, 100 << 20)                            # default 85 % request is capped at 80 %
    assert big.total_size == int((100 << 20) * 0.80)
    a.cleanup()
    assert a.slab_base == 0 and not rt.allocs


# ----------------------------------------------------------------------------- codegen
def test_codegen_sanitises_and_keys_the_cache(tmp_path):
    assert _sanitize_var(32) == "32" and _sanitize_var("abc_1") == "abc_1"
    for bad in ["a b", "x;rm", "1-2", "$(id)", ""]:
        with pytest.raises(CudaSafetyError):
            _sanitize_var(bad)
    with pytest.raises(CudaSafetyError):
        _sanitize_var([1])
    eng = CodegenEngine(cache_dir=tmp_path)
    p0 = eng.cache_path("decode_attention", "sm_100a")
    p1 = eng.cache_path("decode_attention", "sm_100a", split_kv_chunk_size=32)
    p2 = eng.cache_path("decode_attention", "sm_100a", split_kv_chunk_size=16)
    assert len({p0, p1, p2}) == 3 and p0.parent.name == "sm_100a" and re.fullmatch(r"kernel_[0-9a-f]{16}\.cubin", p0.name)
    assert eng.cache_path("decode_attention", "sm_100a") == p0
    with pytest.raises(CudaSafetyError):
        eng.compile_kernel("no_such_template", "sm_100a")
    with pytest.raises(CudaSafetyError):
        eng.compile_kernel("decode_attention", "sm_90a")          # sm_100a only
    with pytest.raises(CudaSafetyError):
        eng.compile_kernel("decode_attention", "gfx1102")


def test_codegen_compiles_and_recompiles_once_on_load_failure(tmp_path):
    eng = CodegenEngine(cache_dir=tmp_path)
    path = eng.compile_kernel("decode_attention", "sm_100a", split_kv_chunk_size=32)
    assert Path(path).stat().st_size > 10_000

    class Flaky:
        def __init__(self): self.calls = 0
        def load_kernel(self, p, name):
            self.calls += 1
            if self.calls == 1:
                raise CudaRuntimeError("stale binary")
            return ("module", name)
    mtime = Path(path).stat().st_mtime_ns
    flaky = Flaky()
    assert eng.load_kernel_safe(flaky, "decode_attention", "sm_100a", "k", split_kv_chunk_size=32) == ("module", "k")
    assert flaky.calls == 2 and Path(path).stat().st_mtime_ns > mtime


def test_every_kernel_of_the_signature_table_is_in_the_cubin():
    """The argument-count table and the cubin must not drift apart: every kernel the table lists has
    a code section of that name in the ahead-of-time cubin, and every exported `vteb_*` /
    reference-named kernel of the cubin is in the table."""
    import re
    from vte_b200.compiler.codegen import CodegenEngine
    data = Path(CodegenEngine().compile_kernel("decode_attention", "sm_100a")).read_bytes()
    for name in KERNEL_SIGNATURES:
        assert b".text." + name.encode() + b"\0" in data, name
    in_cubin = {m.decode() for m in re.findall(rb"\.text\.([A-Za-z0-9_]+_kernel)\0", data)}
    assert in_cubin == set(KERNEL_SIGNATURES), in_cubin ^ set(KERNEL_SIGNATURES)


def test_oom_error_is_a_safety_error():
    assert issubclass(MemoryGuardianOOMError, CudaSafetyError)


def test_balanced_partition_restatement_invariants():
    """Every position of every (sequence, head group) lies in exactly one piece, pieces of a pair get
    consecutive split indices from 0, no pair exceeds its splits, and shares differ by a tile at most
    unless one long sequence forces larger shares."""
    from vte_b200.core.split_kv_attention import balanced_pieces, balanced_split_count
    rng = np.random.default_rng(5)
    for batch, n_hg, lo, hi, tile in ((64, 1, 1024, 16384, 32), (16, 2, 2048, 65536, 32), (8, 1, 1024, 16384, 32),
                                      (2, 2, 2048, 65536, 64), (3, 4, 1, 40, 16), (5, 1, 1, 3, 64)):
        lengths = rng.integers(lo, hi + 1, size=batch)
        C = balanced_split_count(148, batch, n_hg)
        pieces = balanced_pieces(lengths, n_hg, 148, C, tile)
        assert len(pieces) == 148
        cover = {}
        for cta in pieces:
            for (b, h, c, a, e) in cta:
                assert 0 <= c < C and 0 <= a < e <= lengths[b]
                cover.setdefault((b, h), []).append((c, a, e))
        assert len(cover) == batch * n_hg
        for (b, h), lst in cover.items():
            lst.sort()
            assert [c for c, _, _ in lst] == list(range(len(lst)))
            assert lst[0][1] == 0 and lst[-1][2] == lengths[b]
            assert all(lst[i][2] == lst[i + 1][1] for i in range(len(lst) - 1))
        sizes = [sum(e - a for (_, _, _, a, e) in cta) for cta in pieces]
        busy = [s for s in sizes if s]
        assert max(busy) - min(busy[:-1] or busy) <= tile or max(lengths) * n_hg * 148 > (C - 1) * sum(lengths) * n_hg
    # one long sequence among short ones: shares grow so that it still fits its splits
    pieces = balanced_pieces([100000, 10, 10, 10], 1, 148, 8, 32)
    assert max(c for cta in pieces for (_, _, c, _, _) in cta) <= 7
    assert sum(1 for cta in pieces if cta) < 148
