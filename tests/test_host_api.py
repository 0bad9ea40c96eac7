"""Host-side GEMM front-end (no GPU): the reference's own unit tests for this layer, restated against the
C ABI -- src/t0/gemm_gen.rs:544-631 (auto_select sanity, legacy heuristic pins, epilogue name tags,
kernarg layout) -- plus grid arithmetic, presets, the plan resolver and the library's exported symbols."""
import ctypes as C
import os
import re
import struct

import pytest

import t0_gpu_b200 as t
from t0_gpu_b200 import _lib
from t0_gpu_b200.gemm_gen import EpilogueOp, GemmConfig, GemmTranspose

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    with open(os.path.join(ROOT, "include", "t0b200.h")) as f:
        text = f.read()
    declared = set(re.findall(r"T0B_API\s+[\w\s\*]+?\b(t0b_\w+)\s*\(", text))
    assert len(declared) >= 60
    lib = C.CDLL(_lib.LIB_PATH)
    missing = [n for n in sorted(declared) if not hasattr(lib, n)]
    assert not missing, missing
    # the Python binding declares exactly the header's functions
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)


def test_sys_binding_matches_the_header():
    """The Rust `-sys` file a maintainer of the reference crate adds is generated from the header: the committed copy
    (include/t0b200_sys.rs) and the copy embedded in the integration guide at the repository root are both up to date, and every exported function is
    declared in it with as many parameters as the C prototype has."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("make_sys_rs", os.path.join(ROOT, "include", "make_sys_rs.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    text = gen.generate()
    with open(os.path.join(ROOT, "include", "t0b200_sys.rs")) as f:
        assert f.read() == text, "include/t0b200_sys.rs is stale: run python include/make_sys_rs.py"
    guide = os.path.join(ROOT, "INTEGRATION" + ".md")     # the integration guide embeds the binding between two markers
    with open(guide) as f:
        doc = f.read()
    shown = doc.split("<!-- BEGIN t0b200_sys.rs -->\n```rust\n")[1].split("```\n<!-- END t0b200_sys.rs -->")[0]
    assert shown == text, "the binding embedded in the integration guide is stale"
    with open(os.path.join(ROOT, "include", "t0b200.h")) as f:
        header = re.sub(r"/\*.*?\*/", " ", f.read(), flags=re.S)
    protos = re.findall(r"T0B_API\s+[\w\s\*]+?\b(t0b_\w+)\s*\((.*?)\)\s*;", header, flags=re.S)
    assert len(protos) >= 100
    for name, args in protos:
        m = re.search(r"pub fn %s\((.*?)\)( -> [^;]+)?;" % name, text)
        assert m, f"{name} is missing from the -sys binding"
        n_c = 0 if args.strip() in ("", "void") else len(args.split(","))
        n_rs = 0 if not m.group(1).strip() else len(m.group(1).split(", "))
        assert n_c == n_rs, (name, n_c, n_rs)
    assert "is_async: i32" in text and " async:" not in text          # `async` is a Rust keyword


def test_no_gpu_means_loud_failure():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(t.T0Error):
        t.GpuRuntime()


def test_auto_select_sizes():
    """gemm_gen.rs:549-572.  tile_k is 64 on B200 (one 128-byte swizzle row), where the reference pins 16."""
    c = t.auto_select(256, 256, 256)
    assert 16 <= c.tile_m <= 256 and 32 <= c.tile_n <= 128 and c.wg_size >= 32
    c = t.auto_select(1024, 1024, 1024)
    assert c.tile_m >= 64 and c.tile_k == 64
    c = t.auto_select(8192, 8192, 8192)
    assert c.tile_m >= 64
    c = t.auto_select(128, 4096, 4096)
    assert 128 % c.tile_m == 0
    with pytest.raises(ValueError):
        t.auto_select(0, 16, 16)


def _shipped_rows():
    rows = []
    with open(os.path.join(ROOT, "t0_gpu_b200", "csrc", "t0b_tuned_table.inc")) as f:
        for line in f:
            m = re.match(r'\{(\d+), (\d+), (\d+), (\d), (\d), (\d), "(\w+)", (\d+), (\d), (\d+), ([\d.]+)f\},', line.strip())
            if m and int(m.group(1)) > 0:
                rows.append((int(m.group(1)), int(m.group(2)), int(m.group(3)), int(m.group(4)), int(m.group(5)), int(m.group(6)),
                             m.group(7), int(m.group(8)), int(m.group(9)), int(m.group(10))))
    return rows


def test_auto_select_answers_from_the_shipped_table_then_the_cost_model():
    """auto_select = predict_best over the tune cache in the reference (src/t0/cost_model.rs:593-601, 788-1078): here a
    table measured on B200 ships inside the library, and shapes it does not hold fall through to the cost model."""
    rows = _shipped_rows()
    assert len(rows) >= 20 and (8192, 8192, 8192, 0, 0, 0) in [r[:6] for r in rows]      # the benchmark shapes are in it
    for (m, n, k, ta, tb, ob, preset, sk, swap, group) in rows:
        cfg, src = t.auto_select_source(m, k, n, bool(ta), bool(tb), ob)
        want = t.GemmConfig.preset(preset)
        assert src == "table", (m, n, k, src)
        assert (cfg.tile_m, cfg.tile_n, cfg.split_k or 0, int(cfg.swap_grid), cfg.lds_pad) == \
            (want.tile_m, want.tile_n, sk if sk > 1 else 0, swap, group)
    # the layout-less front door prefers the NT / f32 row of a shape
    by_shape = {}
    for r in rows:
        by_shape.setdefault(r[:3], []).append(r)
    for (m, n, k), rs in by_shape.items():
        pick = sorted(rs, key=lambda r: [(0, 1, 0), (0, 0, 0), (1, 0, 0), (1, 1, 0), (0, 1, 1), (0, 0, 1), (1, 0, 1), (1, 1, 1)].index(r[3:6]))[0]
        got = t.auto_select(m, k, n)
        assert (got.tile_m, got.tile_n) == (t.GemmConfig.preset(pick[6]).tile_m, t.GemmConfig.preset(pick[6]).tile_n)
    # a shape nobody measured: the cost model answers
    cfg, src = t.auto_select_source(1000, 3000, 777)
    assert src == "model" and cfg.tile_m >= 128
    with pytest.raises(ValueError):
        t.auto_select_source(0, 1, 1)


def test_auto_select_legacy_preserved():
    """gemm_gen.rs:575-584."""
    c = t.auto_select_legacy(256, 256, 256)
    assert (c.split_k or 1) > 1 and c.tile_m == 64
    c = t.auto_select_legacy(1024, 1024, 1024)
    assert c.tile_m == 128 and c.wgp_mode
    # remaining branches of the 7-branch heuristic
    c = t.auto_select_legacy(128, 4096, 4096)
    assert (c.tile_m, c.tile_n, c.split_k, c.swap_grid) == (128, 64, 4, False)
    c = t.auto_select_legacy(512, 4096, 4096)
    assert (c.tile_m, c.split_k, c.swap_grid) == (128, 8, False)
    c = t.auto_select_legacy(4096, 4096, 4096)
    assert (c.tile_m, c.split_k, c.swap_grid) == (128, 8, True)
    c = t.auto_select_legacy(4032, 4096, 4096)     # 64 | M, 128 does not
    assert (c.tile_m, c.tile_n, c.split_k) == (64, 64, 4)
    c = t.auto_select_legacy(4000, 4096, 4096)     # only 32 | M
    assert (c.tile_m, c.tile_n) == (32, 64)
    # clamp_sk keeps K % (tile_k * sk) == 0
    c = t.auto_select_legacy(256, 48, 256)
    sk = c.split_k or 1
    assert 48 % (16 * sk) == 0


def test_backward_selectors_permute_dims():
    assert t.auto_select_backward_data(1024, 32000, 4096).name() == t.auto_select(1024, 32000, 4096).name()
    assert t.auto_select_backward_weight(1024, 32000, 4096).name() == t.auto_select(32000, 1024, 4096).name()


def test_epilogue_name_tags():
    """gemm_gen.rs:591-602."""
    cfg = GemmConfig.tile_32x64_k16()
    assert "t0_gemm_32x64_k16" in cfg.name() and "_bias" not in cfg.name()
    cfg.epilogue = EpilogueOp.BiasAddStoreF32
    assert cfg.name().endswith("_bias")
    cfg.epilogue = EpilogueOp.BiasAddReluStoreF32
    assert cfg.name().endswith("_bias_relu")


def test_config_names_match_reference_format():
    assert GemmConfig.tile_64x64_k16().name() == "t0_gemm_64x64_k16_ldsdb_wgp"
    assert GemmConfig.tile_32x64_direct().name() == "t0_gemm_32x64_k16_direct_wgp"
    c = GemmConfig.tile_128x128_2pass().with_(split_k=4, swap_grid=False, wgp_mode=False, transpose=GemmTranspose.NN)
    assert c.name() == "t0_gemm_128x64_k16_ldsdb_sk4_2p_mg_nn"
    assert GemmConfig.tile_64x64_k16().with_(split_k=1).name() == "t0_gemm_64x64_k16_ldsdb_wgp"


def test_presets_and_getters():
    c = GemmConfig.tile_128x64_k32()
    assert (c.tile_m, c.tile_n, c.tile_k, c.wg_size) == (128, 64, 32, 128)
    assert c.n_waves() == 4 and c.rows_per_wave() == 32 and c.n_row_blocks() == 2 and c.n_col_tiles() == 4
    assert c.k_sub_steps() == 2 and c.lds_per_buffer() == (128 + 64) * 32 * 2 and c.lds_total() == 2 * c.lds_per_buffer()
    # estimated_vgprs: acc 2*4*8 + x_frag 16 + wt_frag 32 + gmem (4+2... per thread loads) + 49
    assert c.estimated_vgprs() == 2 * 4 * 8 + 2 * 8 + 4 * 8 + (128 * 32 * 2 // 128 // 16) * 4 + (64 * 32 * 2 // 128 // 16) * 4 + 49
    assert c.is_feasible()
    assert len(t.sweep_configs()) == 9 and len(t.standard_configs()) == 14
    assert t.standard_configs()[8].split_k == 4 and t.standard_configs()[8].tile_m == 16
    with pytest.raises(ValueError):
        GemmConfig.preset("nope")


def test_kernargs_layouts():
    """gemm_gen.rs:414-456, 619-630; tile_ir.rs:3173-3190."""
    cfg = GemmConfig.tile_32x64_k16()
    ka = t.build_kernargs_with_bias(0x1000, 0x2000, 0x3000, 64, 64, 128, cfg, 0x4000)
    assert len(ka) == 48 and struct.unpack_from("<Q", ka, 40)[0] == 0x4000
    ka = t.build_kernargs(0x1122334455667788, 0x2000, 0x3000, 96, 160, 128, cfg)
    x, wt, y, k, n, z, stride = struct.unpack("<QQQIIII", ka)
    assert (x, wt, y, k, n, z, stride) == (0x1122334455667788, 0x2000, 0x3000, 96, 160, 0, 0)
    ka = t.build_kernargs(1, 2, 3, 96, 160, 128, cfg.with_(split_k=4))
    assert struct.unpack_from("<I", ka, 36)[0] == 128 * 160 * 4
    ka = t.build_kernargs_m(1, 2, 3, 96, 160, 33)
    assert len(ka) == 44 and struct.unpack_from("<III", ka, 32) == (0, 0, 33)
    # backward helpers permute (k, n, m)
    ka = t.build_kernargs_backward_data(1, 2, 3, 128, 512, 256, cfg)       # K_contract = N_orig, N_out = K_orig
    assert struct.unpack_from("<II", ka, 24) == (512, 256)
    ka = t.build_kernargs_backward_weight(1, 2, 3, 128, 512, 256, cfg)     # K_contract = M, N_out = K_orig
    assert struct.unpack_from("<II", ka, 24) == (128, 256)


def test_grids():
    """gemm_gen.rs:286-309, 402-409: x is in threads, split-K multiplies the slow axis."""
    c = GemmConfig.tile_128x64_k16()
    assert t.compute_grid(c, 256, 256) == (4 * 128, 2)
    assert t.compute_grid(c.with_(swap_grid=False), 256, 256) == (2 * 128, 4)
    assert t.compute_grid(c, 129, 65) == (2 * 128, 2)                       # ceiling division
    assert t.compute_grid(GemmConfig.tile_128x128_2pass(), 256, 256) == (2 * 128, 2)   # 2 column passes
    assert t.compute_grid_split_k(c, 256, 256, 4) == (4 * 128, 8)
    assert t.compute_grid_auto(c.with_(split_k=8), 256, 256) == (4 * 128, 16)
    assert t.compute_grid_auto(c, 256, 256) == t.compute_grid(c, 256, 256)
    with pytest.raises(AssertionError):
        t.compute_grid_split_k(c, 256, 256, 3)                               # the reference asserts a power of 2
    assert t.compute_grid_backward_data(c, 256, 512) == t.compute_grid_auto(c, 256, 512)
    assert t.compute_grid_backward_weight(c, 1024, 512) == t.compute_grid_auto(c, 1024, 512)


def test_plan_resolution():
    p = t.resolve_plan(None, 8192, 8192, 8192)
    assert (p.bm, p.bn, p.bk, p.cta_group, p.m_tiles, p.n_tiles) == (256, 512, 64, 2, 1, 2) and p.use_tma and p.smem_bytes <= 227 * 1024
    p = t.resolve_plan(GemmConfig.preset("b200_512x256"), 8192, 8192, 8192)
    assert (p.bm, p.bn, p.cta_group, p.m_tiles, p.n_tiles, p.stages) == (512, 256, 2, 2, 1, 4)
    p = t.resolve_plan(GemmConfig.preset("b200_256x256"), 8192, 8192, 8192)
    assert (p.bm, p.bn, p.cta_group, p.m_tiles, p.stages) == (256, 256, 2, 1, 6)
    # reference presets run as single-CTA 128-row tiles
    p = t.resolve_plan(GemmConfig.tile_64x64_k16().with_(split_k=4), 256, 256, 256)
    assert (p.bm, p.bn, p.cta_group, p.split_k, p.kb_per_split) == (128, 64, 1, 4, 1)
    # more slabs than 64-wide K blocks: effective split shrinks
    p = t.resolve_plan(GemmConfig.tile_64x64_k16().with_(split_k=8), 64, 64, 256)
    assert p.split_k == 4
    # a row pitch that is not a multiple of 16 bytes cannot be addressed by TMA
    assert not t.resolve_plan(None, 33, 50, 100, lda=100, ldb=100).use_tma
    assert t.resolve_plan(None, 33, 50, 100, lda=104, ldb=104).use_tma
    # B200-native presets
    p = t.resolve_plan(GemmConfig.preset("b200_128x256"), 4096, 4096, 4096)
    assert (p.bm, p.bn, p.cta_group, p.stages) == (128, 256, 1, 4)
    for name in ("b200_128x64", "b200_128x128", "b200_128x256", "b200_256x128", "b200_256x256", "b200_512x256", "b200_256x512"):
        p = t.resolve_plan(GemmConfig.preset(name), 4096, 4096, 4096)
        assert p.smem_bytes <= 227 * 1024 and p.stages >= 4


def test_split_k_selected_for_small_grids():
    c = t.auto_select(512, 16384, 512)
    assert (c.split_k or 1) >= 4
    assert t.auto_select(8192, 8192, 8192).split_k is None
    assert _lib.lib().t0b_gemm_workspace_bytes(C.byref(c.to_c()), 512, 512, 16384) == (c.split_k) * 512 * 512 * 4


def test_cost_model_split_k_paths_for_unmeasured_skinny_shapes():
    """Shapes outside the shipped table: the model's split-K costs come from in-kernel timer measurements (cluster
    exchange ~7000 cycles, slab round trip + second kernel ~14000 + bytes), so skinny shapes that fit one wave of
    clusters take the one-launch cluster path (single-CTA tile, at most 8 K ranges) -- what the on-device tuner picks
    for them -- and only deeper splits fall back to slabs."""
    for (m, k, n) in ((256, 4096, 256), (16, 4096, 4096), (128, 8192, 8192), (1024, 8192, 1024)):
        cfg, src = t.auto_select_source(m, k, n)
        assert src == "model", (m, k, n, src)
        assert cfg.tile_m == 128 and 2 <= (cfg.split_k or 1) <= 8, (m, k, n, cfg.name())
    # A full grid needs no split at all, however deep K is.
    assert t.auto_select_source(4096, 16384, 4096)[0].split_k is None


def test_autotune_cache_roundtrip(tmp_path):
    """src/t0/auto_gemm.rs:578-610: save + load of the per-shape JSON cache, and a file in the reference's own
    format (as its `save_cache` writes it) parses to the same config."""
    d = str(tmp_path / "t0_autotune_cache_test").encode()
    L = _lib.lib()
    cfg = GemmConfig.tile_128x64_k32()
    assert L.t0b_tune_cache_save(d, 4096, 4096, 4096, C.byref(cfg.to_c()), 79.2) == 0
    out = _lib.GemmConfigC()
    tf = C.c_float()
    assert L.t0b_tune_cache_load(d, 4096, 4096, 4096, C.byref(out), C.byref(tf)) == 0
    got = GemmConfig.from_c(out)
    assert (got.tile_m, got.tile_n, got.tile_k, got.wg_size) == (128, 64, 32, 128)
    assert abs(tf.value - 79.2) < 0.1 and got.split_k is None and got.wgp_mode and got.swap_grid
    text = open(os.path.join(d.decode(), "gemm_4096x4096x4096.json")).read()
    assert text.startswith('{"tile_m":128,"tile_n":64,"tile_k":32,"wg_size":128,"split_k":1,"lds_pad":0,"n_col_passes":1,'
                           '"wgp":true,"swap":true,"tflops":79.20,"all":[["t0_gemm_128x64_k32_ldsdb_wgp",79.20]')
    # a file written by the reference (two entries in "all", split_k 4, swap false)
    with open(os.path.join(d.decode(), "gemm_512x512x16384.json"), "w") as f:
        f.write('{"tile_m":64,"tile_n":64,"tile_k":16,"wg_size":64,"split_k":4,"lds_pad":0,"n_col_passes":1,'
                '"wgp":true,"swap":false,"tflops":14.25,"all":[["t0_gemm_64x64_k16_ldsdb_sk4_mg_wgp",14.25],["x",1.00]]}')
    assert L.t0b_tune_cache_load(d, 512, 512, 16384, C.byref(out), C.byref(tf)) == 0
    got = GemmConfig.from_c(out)
    assert (got.tile_m, got.split_k, got.swap_grid, got.wgp_mode) == (64, 4, False, True) and abs(tf.value - 14.25) < 1e-3
    assert got.name() == "t0_gemm_64x64_k16_ldsdb_sk4_mg_wgp"
    # invalidate removes the entry; loading a missing entry fails
    assert L.t0b_tune_cache_invalidate(d, 4096, 4096, 4096) == 0
    assert L.t0b_tune_cache_load(d, 4096, 4096, 4096, C.byref(out), C.byref(tf)) != 0


def test_gemm_tuner_bookkeeping(tmp_path, capsys):
    """GemmTuner's cache layers without a device (src/t0/auto_gemm.rs:325-417, test :581-610): a result saved in the
    reference's JSON format is found by a fresh tuner as a `from_cache` entry, `invalidate` removes the memory and
    the disk entry, `clear` removes the directory."""
    from t0_gpu_b200.auto_gemm import GemmTuner, global_tuner

    class FakeRuntime:                      # stands where the device would measure
        handle = None
        measured = 0

        def _check(self, rc):
            pass

        def tune(self, m, n, k):
            FakeRuntime.measured += 1
            return GemmConfig.preset("b200_256x256"), 1234.5

    d = tmp_path / "tuner"
    tuner = GemmTuner.with_cache_dir(str(d))
    assert tuner.max_candidates == 8 and tuner.n_iters == 5 and tuner.cache == {}
    assert tuner.cache_path(4096, 1024, 512).endswith("gemm_4096x1024x512.json")
    assert tuner.load_cache(64, 64, 64) is None
    cfg = GemmConfig.preset("128x64_k16").with_(split_k=4, swap_grid=False)
    assert _lib.lib().t0b_tune_cache_save(str(d).encode(), 64, 64, 64, C.byref(cfg.to_c()), 42.25) == 0
    got = tuner.tune(FakeRuntime(), 64, 64, 64)                      # disk hit
    assert (got.tile_m, got.tile_n, got.split_k, got.swap_grid) == (128, 64, 4, False)
    r = tuner.cache[(64, 64, 64)]
    assert r.from_cache and abs(r.best_tflops - 42.25) < 1e-3 and r.key == (64, 64, 64) and r.all == []
    n_before = FakeRuntime.measured
    assert tuner.tune(FakeRuntime(), 64, 64, 64) == got              # memory hit: the runtime is not asked again
    assert FakeRuntime.measured == n_before
    best = tuner.tune(FakeRuntime(), 128, 128, 128)                  # miss: measured
    assert best.tile_m == 256 and not tuner.cache[(128, 128, 128)].from_cache
    assert tuner.cache[(128, 128, 128)].all == [(best.name(), 1234.5)]
    tuner.report()
    text = capsys.readouterr().err
    assert "2 entries" in text and "[cached]" in text and "[measured]" in text
    tuner.invalidate(64, 64, 64)
    assert (64, 64, 64) not in tuner.cache and tuner.load_cache(64, 64, 64) is None
    tuner.clear()
    assert tuner.cache == {} and not d.exists()
    assert global_tuner() is global_tuner()


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` needs no GPU: it times the CPU restatement on a bounded sample and prints one JSON
    line with the keys the measurement contract names."""
    import json
    import subprocess
    import sys

    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "bf16 GEMM TFLOP/s" and line["unit"] == "TFLOP/s"
    assert line["value"] > 0 and line["steps"] == 1 and line["higher_is_better"] is True
    assert line["config"]["workload"] == "square_8192_nn_f32out"
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert abs(line["e2e"]["value"] - line["value"]) < 1e-12
