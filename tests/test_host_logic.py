"""Host-side logic that needs no GPU: config records, search-space enumeration and feasibility, cache
round trip, the reference's import names, and that the C-ABI library loads and exports every symbol its
header declares."""
import ctypes
import json
import os
import re

import pytest
import torch

from attention_autotuner_b200.arch import A100, B200, RTX4090, Arch
from attention_autotuner_b200.autotuner.configs import AttnConfig, BaseConfig, supported_configs
from attention_autotuner_b200.autotuner.runtime import KernelError, Runtime, nvcc_command
from attention_autotuner_b200.autotuner.tunner import AttnTunner

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_arch_fields():
    b = B200()
    assert isinstance(b, Arch) and b.compute_capability == "100a"
    assert b.smem_cap == 227 * 1024 and b.tmem_columns == 512 and b.compute_max_core == 148
    for a in (A100(), RTX4090()):
        for f in ("reg_cap", "smem_cap", "compute_max_core", "warp_size", "sm_partition", "transaction_size",
                  "max_smem_usage", "bandwidth", "platform", "compute_capability", "register_per_thread"):
            assert hasattr(a, f)


def test_only_sm100_is_a_build_target():
    with pytest.raises(KernelError):
        nvcc_command(A100(), "x.cu", "x.so")
    cmd = nvcc_command(B200(), "x.cu", "x.so")
    assert "-gencode=arch=compute_100a,code=sm_100a" in cmd


def test_attn_config_legacy_and_new_arguments():
    # the reference's positional form (python/tests/test_runtime.py builds configs this way)
    c = AttnConfig(64, 32, 256, 128, 256, 32, 1, 1, 128, 1, warps_mma1_n=1, warps_mma_n=2)
    c.set_fuse_type("shared")
    assert c.fuse_type == "tmem" and c.Br == 128 and c.Bc == 128 and c.q_tiles == 1
    c2 = AttnConfig(256, 128, 128, 128, q_tiles=2, kv_stages=4, dtype="bf16")
    assert str(c2) == "attn_tmem_256_128_128_128_2_4_128_1_0_1_0_bf16"
    assert c2.tmem_columns() == 512 and c2.smem_bytes() <= B200().smem_cap
    d = json.loads(json.dumps(c2.__dict__))
    c3 = supported_configs[d["operation"]].from_dict(d)
    assert c3 == c2 and repr(c3) == repr(c2)
    assert AttnConfig(128, 128, 128, 512).dv_chunk == 256 and AttnConfig(128, 128, 64, 192).dv_chunk == 64


def _tensors(dqk, dv, dt=torch.float16):
    q = torch.zeros(1, 1, 128, dqk, dtype=dt)
    v = torch.zeros(1, 1, 128, dv, dtype=dt)
    return [q, q, v, v]


def test_attn_search_space_is_feasible():
    arch = B200()
    for dqk, dv in ((64, 64), (128, 128), (256, 256), (256, 512), (128, 64)):
        t = AttnTunner(arch, _tensors(dqk, dv))
        cfgs = t.get_tuned_configs()
        assert cfgs, (dqk, dv)
        for c in cfgs:
            assert c.smem_bytes() <= arch.smem_cap and c.tmem_columns() <= 512
            assert c.Kd == dqk and c.D == dv and dv % c.dv_chunk == 0
        assert len({str(c) for c in cfgs}) == len(cfgs)
        assert t.validate_kernel(t.default_config())
    # two ping-ponging query tiles do not fit tensor memory at dv chunk 256
    assert not AttnTunner(arch, _tensors(128, 256)).validate_kernel(AttnConfig(256, 128, 128, 256, q_tiles=2, kv_stages=2))


def test_cache_round_trip(tmp_path, monkeypatch):
    monkeypatch.setenv("ATTN_B200_CACHE_DIR", str(tmp_path))
    t = AttnTunner(B200(), _tensors(128, 128, torch.bfloat16), causal=True)
    assert t.check_cache() is None
    cfg = AttnConfig(256, 128, 128, 128, q_tiles=2, kv_stages=3, dtype="bf16")
    with open(t._cache_file(), "w") as f:
        json.dump(cfg.__dict__, f)
    assert os.path.basename(t._cache_file()) == "best_config_attention_128_128_sm100a_bf16_causal.json"
    got = t.check_cache()
    assert got == cfg and got.kv_stages == 3
    # tune() returns the cached config without touching a GPU
    assert t.tune() == cfg
    # a cache entry written for another dtype is not used
    assert AttnTunner(B200(), _tensors(128, 128, torch.float16), causal=True).check_cache() is None


def test_tune_without_search_returns_default(monkeypatch, tmp_path):
    monkeypatch.setenv("ATTN_B200_CACHE_DIR", str(tmp_path))
    t = AttnTunner(B200(), _tensors(64, 64))
    assert t.tune(search=False) == t.default_config()


def test_reference_import_names():
    from attention_autotuner_b200 import compat
    compat.install()
    from arch import B200 as B  # noqa: F401
    from autotuner.configs import AttnConfig as C  # noqa: F401
    from autotuner.runtime import Runtime as R, compile_parallel  # noqa: F401
    from autotuner.tunner import AttnTunner as T  # noqa: F401
    from ops.attention_interface import flash_attn_func  # noqa: F401
    from utils.misc import is_close_my  # noqa: F401
    from utils.ref_op import attention_ref, retnet_ref  # noqa: F401
    assert C is AttnConfig


def test_library_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "attn_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    names = re.findall(r"\b(attn_b200_\w+)\s*\(", header)
    assert len(names) >= 6
    for n in set(names):
        assert hasattr(lib, n), n
    assert lib.attn_b200_abi_version() >= 1
    assert lib.attn_b200_last_error() is not None


def test_argument_validation_without_gpu(lib):
    # rejected before any CUDA call
    rc = lib.attn_b200_fa_fwd(None, None, None, None, None, 1, 1, 128, 128, 128, 128, 0, 0.1, 0, None)
    assert rc == 1 and b"null" in lib.attn_b200_last_error()
    buf = ctypes.create_string_buffer(64)
    p = ctypes.cast(buf, ctypes.c_void_p)
    assert lib.attn_b200_fa_fwd(p, p, p, p, None, 1, 1, 128, 128, 96, 128, 0, 0.1, 0, None) == 2   # dqk not built
    assert lib.attn_b200_fa_fwd(p, p, p, p, None, 1, 1, 128, 128, 128, 128, 7, 0.1, 0, None) == 1  # dtype
    assert lib.attn_b200_fa_fwd(p, p, p, p, None, 0, 1, 128, 128, 128, 128, 0, 0.1, 0, None) == 1  # B
    assert lib.attn_b200_fa_fwd(p, p, p, p, None, 1, 1, 128, 128, 128, 128, 0, -1.0, 0, None) == 1  # scale
    # attention backward: (q,k,v,o,do,lse,dq,dk,dv, B,H,Lq,Lkv,d, dtype, scale, causal, stream)
    rc = lib.attn_b200_fa_bwd(p, p, p, None, p, p, p, p, p, 1, 1, 128, 128, 128, 0, 0.1, 0, None)
    assert rc == 1 and b"null" in lib.attn_b200_last_error()
    assert lib.attn_b200_fa_bwd(p, p, p, p, p, p, p, p, p, 1, 1, 128, 128, 96, 0, 0.1, 0, None) == 2    # head dimension
    assert lib.attn_b200_fa_bwd(p, p, p, p, p, p, p, p, p, 1, 1, 128, 256, 128, 0, 0.1, 1, None) == 2   # causal, Lq != Lkv
    assert lib.attn_b200_fa_bwd(p, p, p, p, p, p, p, p, p, 1, 1, 128, 128, 128, 3, 0.1, 0, None) == 1   # dtype
    assert lib.attn_b200_fa_bwd(p, p, p, p, p, p, p, p, p, 1, 0, 128, 128, 128, 0, 0.1, 0, None) == 1   # H


def test_chunkwise_segments_and_their_scratch_without_gpu(lib):
    """Host arithmetic of the segmented chunkwise RetNet: how many segments the library prefers (as many as fill 148 SMs
    with CTAs of 128 columns, each at least four chunks long; none when the slices alone fill the GPU or dv is not a
    multiple of 128), how a forced count maps onto whole chunks, and the scratch (one fp32 [dqk x dv] tile per slice
    and segment but the last). Argument errors are rejected before any CUDA call."""
    ws = lib.attn_b200_ret_chunk_workspace_bytes
    tile = 256 * 512 * 4
    assert ws(1, 8, 16384, 256, 512, 0) == 3 * 8 * tile          # 32 tiles of 128 columns -> 4 segments of 32 chunks
    assert ws(8, 8, 2048, 256, 512, 0) == 0                      # 256 tiles: the slices fill the GPU
    assert ws(1, 2, 4096, 256, 256, 0) == 7 * 2 * 256 * 256 * 4  # 4 tiles, 32 chunks: 8 segments of 4 chunks
    assert ws(1, 1, 512, 256, 512, 0) == 0                       # four chunks: nothing to cut
    assert ws(1, 8, 16384, 256, 192, 0) == 0                     # dv not a multiple of 128: no preference
    assert ws(1, 3, 1100, 128, 128, 1) == 0
    for asked, count in ((2, 2), (3, 3), (4, 3), (5, 5), (9, 9), (50, 9)):   # nine chunks: ceil(9 / asked) chunks per segment
        assert ws(1, 3, 1100, 128, 128, asked) == (count - 1) * 3 * 128 * 128 * 4, asked
    assert ws(0, 1, 128, 128, 128, 0) == 0 and ws(1, 1, 128, 128, 128, -1) == 0
    buf = ctypes.create_string_buffer(256)
    p = ctypes.c_void_p((ctypes.addressof(buf) + 63) & ~63)      # the checks want 16- and 32-byte aligned tensors
    call = lambda **kw: lib.attn_b200_ret_chunk_fwd_ws(p, p, p, p, p, kw.get("w"), kw.get("nbytes", 0), kw.get("segments", 0),
                                                     1, 1, kw.get("L", 1100), kw.get("dqk", 128), 128, 0, 1.0, None)
    assert call(dqk=64) == 2
    assert call(segments=-1) == 1
    assert call(segments=3) == 1 and b"scratch" in lib.attn_b200_last_error()          # no scratch at all
    assert call(segments=3, w=p, nbytes=64) == 1 and b"scratch" in lib.attn_b200_last_error()


def test_per_config_library_builds_and_exports_reference_symbols(tmp_path):
    cfg = AttnConfig(128, 128, 64, 64, q_tiles=1, kv_stages=2)
    rt = Runtime(B200(), cfg, tmp_dir=str(tmp_path))
    assert rt.libname.startswith(str(cfg) + "_") and rt.libname.endswith(".so")
    so = ctypes.CDLL(rt.lib_path)
    for n in ("kernel_entry", "profile", "kernel_entry_ex", "profile_ex", "last_error", "device_status"):
        assert hasattr(so, n)
    # second construction reuses the file
    mtime = os.path.getmtime(rt.lib_path)
    assert Runtime(B200(), cfg, tmp_dir=str(tmp_path)).libname == rt.libname
    assert os.path.getmtime(rt.lib_path) == mtime
    with pytest.raises(KernelError):
        rt.apply([torch.zeros(1, 1, 128, 64, dtype=torch.float16)] * 4)  # CPU tensors: no CPU path


def test_host_buffer_operators_need_a_gpu_and_split_the_batch_evenly():
    from attention_autotuner_b200.ops import host_interface as hi
    assert hi._bounds(5, 2) == [(0, 3), (3, 5)]
    assert hi._bounds(3, 10) == [(0, 1), (1, 2), (2, 3)]
    assert hi._pieces(2, 4, None) == [(0, 1, 0, 4), (1, 2, 0, 4)]
    assert hi._pieces(2, 4, 4) == [(0, 1, 0, 2), (0, 1, 2, 4), (1, 2, 0, 2), (1, 2, 2, 4)]
    assert hi._pieces(1, 3, None) == [(0, 1, 0, 1), (0, 1, 1, 2), (0, 1, 2, 3)]
    assert hi._pieces(4, 3, 2) == [(0, 2, 0, 3), (2, 4, 0, 3)]
    assert hi._pieces(2, 1, None) == [(0, 1, 0, 1), (1, 2, 0, 1)]
    assert hi._pieces(1, 5, 100) == [(0, 1, h, h + 1) for h in range(5)]
    import torch
    if not torch.cuda.is_available():
        x = torch.zeros(1, 1, 128, 64, dtype=torch.float16)
        with pytest.raises(RuntimeError, match="no CPU path"):
            hi.flash_attn_host(x, x, x, None)


def test_prune_stale_removes_only_libraries_of_other_source_hashes(tmp_path):
    from attention_autotuner_b200.autotuner.runtime import prune_stale, source_tag
    keep = tmp_path / f"attn_x_{source_tag()}.so"
    keep_src = tmp_path / f"attn_x_{source_tag()}.cu"
    old = tmp_path / "attn_x_0123456789.so"
    other = tmp_path / "notes.txt"
    for f in (keep, keep_src, old, other):
        f.write_text("x")
    assert prune_stale(str(tmp_path)) == 1
    assert keep.exists() and keep_src.exists() and other.exists() and not old.exists()


def test_cta_pair_knob_in_configs_and_search_space():
    """CTA pairing is part of every operator's search space; the tuner rejects pair configurations whose tiles cannot
    be split between two CTAs, and the generated launch shim selects the pair kernels."""
    from attention_autotuner_b200.autotuner.configs import RetBwdConfig, RetConfig
    from attention_autotuner_b200.autotuner.runtime import _create_entry_code
    from attention_autotuner_b200.autotuner.tunner import RetBwdTunner, RetTunner
    z = torch.zeros(1, 1, 1, 256, dtype=torch.float16)
    zv = torch.zeros(1, 1, 1, 512, dtype=torch.float16)
    at = AttnTunner(B200(), [torch.zeros(1, 1, 1, 128, dtype=torch.float16)] * 4)
    cfgs = at.get_tuned_configs()
    assert any(c.cta_pair for c in cfgs) and any(not c.cta_pair for c in cfgs)
    assert not at.validate_kernel(AttnConfig(256, 128, 128, 128, q_tiles=2, kv_stages=4, dv_chunk=64, cta_pair=1))
    assert not at.validate_kernel(AttnConfig(128, 128, 128, 128, q_tiles=1, kv_stages=4, dv_chunk=128, cta_pair=1))
    pair = AttnConfig(256, 128, 128, 128, q_tiles=2, kv_stages=4, dv_chunk=128, cta_pair=1)
    assert at.validate_kernel(pair)
    src = _create_entry_code(pair)
    assert "FaPairConfig<128, 8, false>" in src and "fa_fwd_pair_launch<Cfg>" in src
    assert "fa_fwd_launch_auto<Cfg>" in _create_entry_code(AttnConfig(256, 128, 128, 128, q_tiles=2, kv_stages=4, dv_chunk=128))
    # the form of the grid is a knob too: chosen per call by default, or forced
    grid_cfg = AttnConfig(256, 128, 128, 128, q_tiles=2, kv_stages=4, dv_chunk=128, persistent=0)
    pers_cfg = AttnConfig(256, 128, 128, 128, q_tiles=2, kv_stages=4, dv_chunk=128, persistent=1)
    assert "return fa_fwd_launch<Cfg>" in _create_entry_code(grid_cfg)
    assert "return fa_fwd_persist_launch<Cfg>" in _create_entry_code(pers_cfg)
    assert at.validate_kernel(grid_cfg) and at.validate_kernel(pers_cfg)
    assert str(grid_cfg) != str(pers_cfg) != str(AttnConfig(256, 128, 128, 128, q_tiles=2, kv_stages=4, dv_chunk=128))
    assert not at.validate_kernel(AttnConfig(256, 128, 128, 128, q_tiles=2, kv_stages=4, dv_chunk=128, softmax_split=2, persistent=1))
    assert not at.validate_kernel(AttnConfig(128, 128, 128, 128, q_tiles=1, kv_stages=4, dv_chunk=128, persistent=1))
    assert any(getattr(c, "persistent", -1) == 1 for c in cfgs) and any(getattr(c, "persistent", -1) == 0 for c in cfgs)
    assert AttnConfig.from_dict({k: v for k, v in grid_cfg.to_dict().items() if k != "persistent"}).persistent == -1
    rt = RetTunner(B200(), [z, z, zv, None, zv, None], decay=torch.ones(1))
    assert RetConfig(128, 128, 256, 512).cta_pair == 1 and RetConfig(128, 128, 64, 64).cta_pair == 0
    assert not rt.validate_kernel(RetConfig(128, 128, 256, 512, dv_chunk=64, cta_pair=1))
    assert {c.cta_pair for c in rt.get_tuned_configs()} == {0, 1}
    bt = RetBwdTunner(B200(), [z, z, zv, None, zv, None, z, z, zv, None], decay=torch.ones(1))
    assert not bt.validate_kernel(RetBwdConfig(128, 128, 256, 512, dv_chunk=256, dq_chunk=64, cta_pair=1))
    assert "true>(a" in _create_entry_code(RetBwdConfig(128, 128, 256, 512)).replace(" ", "").replace("\n", "") or \
        ", true>" in _create_entry_code(RetBwdConfig(128, 128, 256, 512))
    # a decay mask is lower triangular whatever `causal` says: one cache entry
    assert RetTunner(B200(), [z, z, zv, None, zv, None], causal=True, decay=torch.ones(1))._cache_file() == rt._cache_file()


def test_committed_cache_files_load_on_any_checkout(tmp_path):
    """Every committed best-config file must be usable wherever the package is installed: no absolute path inside,
    the launch-shim source renders from it, and Runtime gets as far as the nvcc command line in an empty directory.
    (The reference stores template_dir in the file, python/autotuner/base_tunner.py:197-208.)"""
    import glob
    from attention_autotuner_b200.autotuner import runtime as rtm
    cache_dir = os.path.join(ROOT, "attention_autotuner_b200", "cache")
    files = sorted(glob.glob(os.path.join(cache_dir, "*.json")))
    assert len(files) >= 5
    for path in files:
        with open(path) as f:
            d = json.load(f)
        for key, val in d.items():
            assert not (isinstance(val, str) and (val.startswith("/") or ":\\" in val)), (path, key, val)
        assert "template_dir" not in d
        cfg = supported_configs[d["operation"]].from_dict(d)
        assert os.path.isfile(os.path.join(cfg.template_dir, "profile_code.py"))
        assert cfg.template_dir.startswith(os.path.join(ROOT, "attention_autotuner_b200", "csrc"))
        src = rtm._create_entry_code(cfg)
        assert 'extern "C" int kernel_entry(' in src and 'extern "C" float profile(' in src
        rt = Runtime(B200(), cfg, tmp_dir=str(tmp_path), libname="pending")  # "pending": do not compile in the constructor
        cmd = nvcc_command(B200(), os.path.join(rt.tmp_dir, str(cfg) + ".cu"), os.path.join(rt.tmp_dir, str(cfg) + ".so"))
        assert cmd[0].endswith("nvcc") and any(a.startswith("-I") and a.endswith("csrc") for a in cmd)
        assert "template_dir" not in cfg.to_dict() and json.dumps(cfg.to_dict())
    # a path smuggled into a cache file never decides which template is executed
    poisoned = dict(d, template_dir="/nonexistent/elsewhere")
    cfg = supported_configs[d["operation"]].from_dict(poisoned)
    assert "/nonexistent" not in cfg.template_dir and rtm._create_entry_code(cfg)


def test_tuner_cache_writer_stores_no_path(tmp_path, monkeypatch):
    monkeypatch.setenv("ATTN_B200_CACHE_DIR", str(tmp_path))
    cfg = AttnConfig(256, 128, 128, 128, q_tiles=2, kv_stages=5)
    assert "template_dir" not in cfg.to_dict() and "template_dir" not in cfg.__dict__
    assert cfg.template_dir.endswith(os.path.join("csrc", "kernels", "attention"))


def test_library_staleness_is_decided_by_a_source_hash(tmp_path, monkeypatch):
    from attention_autotuner_b200 import build
    fake = tmp_path / "libattn_b200.so"
    monkeypatch.setattr(build, "LIB_PATH", str(fake))
    assert build.is_stale()                       # no library
    fake.write_bytes(b"x")
    assert build.is_stale()                       # library without a stamp
    (tmp_path / "libattn_b200.so.srchash").write_text(build.source_hash() + "\n")
    assert not build.is_stale()
    os.utime(fake, (1, 1))                        # file times do not matter (a fresh checkout has arbitrary ones)
    assert not build.is_stale()
    (tmp_path / "libattn_b200.so.srchash").write_text("0" * 40 + "\n")
    assert build.is_stale()                       # built from other sources


def test_operator_argument_checks_raise_before_any_launch():
    """Mismatched tensors must raise ValueError instead of reaching a kernel that indexes raw pointers."""
    from attention_autotuner_b200.ops import _checks
    from attention_autotuner_b200.ops.attention_interface import flash_attn_func
    from attention_autotuner_b200.ops.retnet_interface import RetNetAttnFunc
    h = torch.float16
    q = torch.zeros(2, 4, 128, 128, dtype=h)
    k = torch.zeros(2, 4, 256, 128, dtype=h)
    v = torch.zeros(2, 4, 256, 128, dtype=h)
    bad = [
        (q, k[:, :2], v, "batch/heads"),                          # fewer k heads (grouped-query layout)
        (q, k, v[:, :2], "batch/heads"),
        (q, k[..., :64], v, "head dimension"),                    # k head dim differs from q
        (q, k, v[:, :, :128], "keys"),                            # v shorter than k
        (q, k.to(torch.bfloat16), v, "dtype"),
        (q.float(), k.float(), v.float(), "float16 or bfloat16"),
        (q[0], k[0], v[0], "4-d"),
        (q[..., :96], k[..., :96], v, "CUDA device" if not torch.cuda.is_available() else "multiple of 64"),
    ]
    for qq, kk, vv, msg in bad:
        with pytest.raises(ValueError, match=msg):
            flash_attn_func(qq, kk, vv, B200())
        with pytest.raises(ValueError, match=msg):
            RetNetAttnFunc(qq, kk, vv, None, B200(), decay=torch.ones(4))
    if not torch.cuda.is_available():
        with pytest.raises(ValueError, match="CUDA device"):
            flash_attn_func(q, k, v, B200())
    # mask / decay forms
    with pytest.raises(ValueError, match="either a mask"):
        _checks.check_mask_decay("op", q, k, None, None)
    with pytest.raises(ValueError, match="either a mask"):
        _checks.check_mask_decay("op", q, k, torch.zeros(4, 128, 256, dtype=h), torch.ones(4))
    with pytest.raises(ValueError, match="mask has shape"):
        _checks.check_mask_decay("op", q, k, torch.zeros(4, 128, 128, dtype=h), None)
    with pytest.raises(ValueError, match="mask has dtype"):
        _checks.check_mask_decay("op", q, k, torch.zeros(4, 128, 256), None)
    with pytest.raises(ValueError, match="per-head"):
        _checks.check_mask_decay("op", q, k, None, torch.ones(3))
    _checks.check_mask_decay("op", q, k, torch.zeros(4, 128, 256, dtype=h), None)
    with pytest.raises(ValueError, match="dO has shape"):
        _checks.check_like("op", "dO", torch.zeros(2, 4, 128, 64, dtype=h), (2, 4, 128, 128), h, q.device)


def test_timing_statistics():
    from attention_autotuner_b200.utils import timing
    s = timing.summarize([5.0, 1.0, 3.0, 2.0, 4.0])
    assert s["median_ms"] == 3.0 and s["min_ms"] == 1.0 and s["reps"] == 5
    assert abs(s["p20_ms"] - 1.8) < 1e-9 and abs(s["p80_ms"] - 4.2) < 1e-9
    assert timing.percentile([7.0], 0.8) == 7.0
    with pytest.raises(ValueError):
        timing.percentile([], 0.5)


def test_bench_flop_model_and_workload_table():
    import bench
    assert abs(bench.flops_of("C2") - 1.0995e12) / 1.0995e12 < 1e-3
    assert abs(bench.flops_of("C5sq") - 70.37e12) / 70.37e12 < 1e-3
    assert abs(bench.flops_of("C5dec") - 4.398e12) / 4.398e12 < 1e-3
    assert abs(bench.flops_of("C5sq", 64) * 8 - bench.flops_of("C5sq")) < 1.0     # 64 of 512 slices on each of 8 ranks
    assert bench.flops_of("C2bwd") == bench.flops_of("C2") * 3.5
    for name in bench.EXTRA_SHORT + bench.STRONG + bench.SUSTAINED:
        assert name in bench.WORKLOADS


def test_cost_model_ranks_the_measured_best_near_the_top():
    """The cost model is fitted on the committed search logs. Held-out check: fit on all logs but one, rank the
    held-out log's candidates; timing only the five predicted fastest must find a configuration within 3 % of the
    exhaustive search's best, for every committed log."""
    from attention_autotuner_b200.autotuner import cost_model as cm
    logs = cm.load_logs()
    assert len(logs) >= 5
    recs = cm.pruning_report(top_k=5, logs=logs)
    assert {r["operation"] for r in recs} == {"attn", "ret", "ret_bwd"}
    for r in recs:
        assert r["regret"] <= 0.03, r
    # the committed weights are the fit of the committed logs, and predictions are in the right range
    w = cm.load_weights()
    refit = cm.fit(logs)
    for op in refit:
        for name, val in refit[op].items():
            assert abs(w[op][name] - val) <= 1e-6 + 1e-6 * abs(val), (op, name)
    name, op, problem, rows = logs[0]
    for cfg, ms in rows:
        assert 0.5 * ms < cm.predict_ms(op, cfg, problem) < 2.0 * ms


def test_cost_model_prunes_the_search_space_without_a_gpu():
    from attention_autotuner_b200.autotuner import cost_model as cm
    t = AttnTunner(B200(), [torch.zeros(8, 16, 4096, 128, dtype=torch.float16)] * 4)
    cfgs = t.get_tuned_configs()
    ranked = cm.rank("attn", cfgs, t.problem())
    assert len(ranked) == len(cfgs) and set(map(str, ranked)) == set(map(str, cfgs))
    # two ping-ponging query tiles beat one, full-width V chunks beat half-width ones
    assert ranked[0].q_tiles == 2 and ranked[0].dv_chunk == 128
    assert ranked[-1].dv_chunk == 64
    assert cm.parse_config_repr("Config(fuse_type=tmem, Br=128, q_tiles=2, dtype=fp16)") == {
        "fuse_type": "tmem", "Br": 128, "q_tiles": 2, "dtype": "fp16"}
    rec = t._cost_model_record({cfgs[0]: 1.0, cfgs[1]: 2.0, cfgs[2]: 0.5}, {cfgs[0]: 1.1, cfgs[1]: 1.9, cfgs[2]: 0.6}, 30, None,
                               10.0, 12.0, k_report=1)
    assert rec["what_if_regret"] == 0.0 and rec["rank_of_measured_best"] == 1 and rec["what_if_search_time_s"] < 12.0
