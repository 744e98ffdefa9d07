"""CPU: the host side of the library - model.bin container, C ABI surface, KV page allocator."""
import json
import os
import re
import struct
import sys

import numpy as np
import pytest

from helpers import write_model
from mini_llm_cuda_b200.model_file import (ModelSpec, named_spec, periodic_layer_types, synth_weights,
                                           write_model_bin)
from oracle.model_bin import read_model_bin

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def api(built_lib):
    from mini_llm_cuda_b200 import api as _api
    return _api


def declared_functions(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mlb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(api):
    L = api.lib()
    names = declared_functions("mlb.h") + declared_functions("mini_llm_compat.h")
    assert len(names) > 40
    for n in names:
        assert hasattr(L, n), f"{n} is declared in include/ but not exported"
    assert b"sm_100a" in L.mlb_version()


def test_reference_named_entry_points_are_exported_with_cxx_linkage():
    """runInferenceLoop & co keep the reference's C++ linkage so that a main written against the
    reference's headers links: check the mangled names in the dynamic symbol table."""
    import subprocess
    from mini_llm_cuda_b200.build import LIB_PATH
    out = subprocess.run(["nm", "-D", "--defined-only", LIB_PATH], capture_output=True, text=True).stdout
    for mangled in ("_Z16runInferenceLoopPKciibb", "_Z12runInferencei", "_Z9loadModelPKc", "_Z9loadVocabPKc",
                    "_Z11vocabLookupPKc", "_Z13vocabGetTokeni", "_Z14allocateMemoryb",
                    "_Z16loadStoryContextPKcii", "_Z23getPreComputedRopeThetaPfi", "seqTokenIndices"):
        assert mangled in out, mangled


def test_no_compute_without_gpu_fails_loudly(api, tmp_path):
    import ctypes as C
    n = C.c_int(0)
    # cudaGetDeviceCount is the first CUDA call of mlb_model_load
    path = write_model(tmp_path, ModelSpec(dim=64, layers=1, heads=1, head_dim=64, ffn_dim=64, vocab=32))
    try:
        m = api.Model(path)
    except api.MlbError as e:
        assert e.status == api.MLB_E_CUDA and "no CPU path" in e.message
    else:
        m.close()      # a GPU is present: loading simply works


def test_writer_reader_round_trip_and_layout(tmp_path):
    spec = named_spec("cfg0")
    w = synth_weights(spec, seed=0)
    path = os.path.join(str(tmp_path), "m.bin")
    write_model_bin(path, spec, w)
    raw = open(path, "rb").read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    assert list(header)[:3] == ["tokenEmbeddings", "finalRMSNormGamma", "transformerBlocks"]
    assert list(header["transformerBlocks"][0])[:9] == [
        "rmsGamma", "queryWeights", "keyWeights", "valueWeights", "outputProjectionWeights", "rmsGamma2",
        "feedForwardWeights1A", "feedForwardWeights1B", "feedForwardWeights2"]
    data_off = 8 + hlen + (8 - (8 + hlen) % 8) % 8
    first = np.frombuffer(raw, dtype="<f4", count=4, offset=data_off)
    assert np.array_equal(first, w["tokenEmbeddings"].ravel()[:4])       # row-major, token row contiguous
    m = read_model_bin(path)
    assert np.array_equal(m["tokenEmbeddings"], w["tokenEmbeddings"])
    for b in range(spec.layers):
        for k, v in w["blocks"][b].items():
            assert np.array_equal(m["blocks"][b][k], v), (b, k)
        for k, v in w["ext"][b].items():
            assert np.array_equal(m["ext"][b][k], v), (b, k)
    # execution order N-1 .. 0: block 0 is the last layer, a delta-net one for cfg0
    assert spec.block_type(0) == "delta_net" and "betaWeights" in m["ext"][0]
    assert m["config"]["layer_types"] == ["attention", "delta_net", "attention", "delta_net"]


def test_converter_gives_a_reference_file_its_config(api, tmp_path):
    """A file as the reference's tools write it (fp32, no config key, QK-norm and gating tensors)
    converted to a bf16 file with an embedded config: the product's own Python reader and the C++
    parser agree with the oracle's reader on it, tensors are the nearest-even bf16 of the source, and
    the command-line form writes the same bytes."""
    import subprocess
    import torch
    from mini_llm_cuda_b200 import model_file as mf
    spec = ModelSpec(dim=128, layers=2, heads=2, head_dim=64, ffn_dim=256, vocab=96, qk_norm=True, query_gating=True)
    w = synth_weights(spec, seed=5, random_gains=True)
    src = os.path.join(str(tmp_path), "ref.bin")
    dst = os.path.join(str(tmp_path), "conv.bin")
    write_model_bin(src, spec, w, with_config=False)
    with pytest.raises(ValueError):
        mf.convert_model_bin(src, dst)                      # heads / head_dim are not in a reference file
    out = mf.convert_model_bin(src, dst, heads=2, head_dim=64, file_dtype="bfloat16", weight_dtype="bfloat16",
                               kv_dtype="bfloat16", rms_eps=1e-8, max_context=256)
    assert out.qk_norm and out.query_gating and out.kv_heads == 2 and out.dim == 128 and out.ffn_dim == 256
    header, got = mf.read_model_bin(dst)
    assert header["config"]["weight_dtype"] == "bfloat16" and header["config"]["max_context"] == 256
    m = read_model_bin(dst)                                  # the oracle's reader
    for k in ("queryWeights", "feedForwardWeights2", "gatedQueryWeights"):
        want = torch.from_numpy(w["blocks"][1][k]).to(torch.bfloat16).float().numpy()
        assert np.array_equal(got["blocks"][1][k], want) and np.array_equal(m["blocks"][1][k], want)
    assert np.array_equal(got["blocks"][0]["queryRMSGamma"], w["blocks"][0]["queryRMSGamma"])     # gains stay fp32
    cfg, nbytes = api.inspect_file(dst)
    assert (cfg.heads, cfg.head_dim, cfg.qk_norm, cfg.query_gating, cfg.max_context) == (2, 64, 1, 1, 256)
    dst2 = os.path.join(str(tmp_path), "conv2.bin")
    r = subprocess.run([sys.executable, "-m", "mini_llm_cuda_b200.model_file", "convert", src, dst2, "--heads", "2",
                        "--head-dim", "64", "--file-dtype", "bfloat16", "--weight-dtype", "bfloat16", "--kv-dtype",
                        "bfloat16", "--max-context", "256"], capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0, r.stderr
    assert open(dst, "rb").read() == open(dst2, "rb").read()


def test_bf16_file_rounding_is_nearest_even(tmp_path):
    import torch
    spec = ModelSpec(dim=64, layers=1, heads=1, head_dim=64, ffn_dim=64, vocab=32)
    w = synth_weights(spec, seed=3)
    path = os.path.join(str(tmp_path), "b.bin")
    write_model_bin(path, spec, w, file_dtype="bfloat16")
    m = read_model_bin(path)
    want = torch.from_numpy(w["tokenEmbeddings"]).to(torch.bfloat16).float().numpy()
    assert np.array_equal(m["tokenEmbeddings"], want)


def test_file_inspect_and_format_errors(api, tmp_path):
    spec = named_spec("cfg0")
    path = write_model(tmp_path, spec, seed=0)
    cfg, n = api.inspect_file(path)
    assert (cfg.dim, cfg.layers, cfg.heads, cfg.head_dim, cfg.ffn_dim, cfg.vocab) == (256, 4, 4, 64, 768, 4096)
    assert cfg.ple_dim == 32 and list(cfg.layer_types[:4]) == [0, 1, 0, 1] and abs(cfg.rms_eps - 1e-5) < 1e-12
    m = read_model_bin(path)
    n_want = m["tokenEmbeddings"].size + m["finalRMSNormGamma"].size + \
        sum(v.size for b in m["blocks"] for v in b.values()) + sum(v.size for b in m["ext"] for v in b.values())
    assert n == n_want
    raw = open(path, "rb").read()

    def expect(blob, status, name):
        p = os.path.join(str(tmp_path), name)
        open(p, "wb").write(blob)
        with pytest.raises(api.MlbError) as e:
            api.inspect_file(p)
        assert e.value.status == status, e.value

    with pytest.raises(api.MlbError) as e:
        api.inspect_file(os.path.join(str(tmp_path), "absent.bin"))
    assert e.value.status == api.MLB_E_IO
    expect(b"", api.MLB_E_FORMAT, "empty.bin")
    expect(raw[:4], api.MLB_E_FORMAT, "short.bin")
    expect(struct.pack("<Q", 10 ** 12) + raw[8:], api.MLB_E_FORMAT, "hugeheader.bin")
    expect(raw[:len(raw) - 100], api.MLB_E_FORMAT, "truncated.bin")                 # data runs past the end
    (hlen,) = struct.unpack("<Q", raw[:8])
    bad = raw[8:8 + hlen].replace(b'"float32"', b'"float16"', 1)
    expect(struct.pack("<Q", len(bad)) + bad + raw[8 + hlen:], api.MLB_E_FORMAT, "dtype.bin")
    expect(struct.pack("<Q", 5) + b"{oops" + b"\0" * 3, api.MLB_E_FORMAT, "json.bin")
    # a reference-format file says nothing about heads: an override is required
    base = write_model(tmp_path, ModelSpec(dim=128, layers=2, heads=2, head_dim=64, ffn_dim=128, vocab=64),
                       name="base.bin", with_config=False)
    with pytest.raises(api.MlbError) as e:
        api.inspect_file(base)
    assert e.value.status == api.MLB_E_INVALID
    cfg, _ = api.inspect_file(base, api.make_override(heads=2, head_dim=64))
    assert cfg.kv_heads == 2 and cfg.qk_norm == 0 and abs(cfg.rms_eps - 1e-8) < 1e-15
    # wrong head count for the tensor shapes
    with pytest.raises(api.MlbError) as e:
        api.inspect_file(base, api.make_override(heads=3, head_dim=64))
    assert e.value.status == api.MLB_E_FORMAT


def test_kv_page_allocator(api):
    a = api.KvAllocator(num_pages=6, batch=3, max_pages_per_seq=4)
    assert a.ensure(0, 0) == 0 and a.table(0) == []
    assert a.ensure(0, 1) == 0 and a.table(0) == [0]
    assert a.ensure(1, 17) == 0 and a.table(1) == [1, 2]
    assert a.ensure(0, 33) == 0 and a.table(0) == [0, 3, 4]       # pages of a sequence need not be contiguous
    assert a.free_pages() == 1
    assert a.ensure(2, 32) == api.MLB_E_KV_FULL                   # needs two, one left: fails, keeps what it got
    assert b"exhausted" in api.lib().mlb_last_error()
    assert a.free_pages() == 0 and a.table(2) == [5]
    assert a.ensure(1, 65) == api.MLB_E_CONTEXT_FULL              # beyond the page table
    a.release(0)
    assert a.free_pages() == 3 and a.table(0) == []
    assert a.ensure(2, 32) == 0 and len(a.table(2)) == 2
    assert a.ensure(5, 1) == api.MLB_E_INVALID


def test_rope_table_bitwise_equals_oracle(api):
    from oracle.decode_oracle import rope_table
    for L, hd, base in ((256, 64, 10000.0), (1024, 128, 10000.0), (64, 64, 500000.0)):
        assert np.array_equal(api.rope_table(L, hd, base), rope_table(L, hd, base))
    t = api.rope_table(4, 64, 10000.0)
    assert np.all(t[0, 0::2] == 1.0) and np.all(t[0, 1::2] == 0.0)      # position 0: cos 1, sin 0
    assert abs(t[1, 0] - np.cos(1.0)) < 1e-7 and abs(t[1, 1] - np.sin(1.0)) < 1e-7


def test_pool_sharding_matches_the_python_sharding_and_refuses_bad_arguments(api):
    """Host side of the multi-GPU pool without a GPU: the C shard ranges are those of the torchrun driver's
    shard_range (contiguous, the first n % world shards one longer, together covering every sequence once),
    and mlb_pool_new turns down argument errors before it touches a device."""
    import ctypes as C
    from mini_llm_cuda_b200.sharding import shard_range
    for n in (0, 1, 7, 8, 64, 255, 256):
        for world in (1, 2, 3, 4, 8):
            cover = []
            for r in range(world):
                got = api.shard_range_c(n, world, r)
                assert got == shard_range(n, world, r)
                cover += list(range(*got))
            assert cover == list(range(n))
    with pytest.raises(api.MlbError):
        api.shard_range_c(8, 4, 4)
    with pytest.raises(api.MlbError):
        api.shard_range_c(8, 0, 0)
    L = api.lib()
    h = C.c_void_p()
    dev = np.array([0, -1], dtype=np.int32)
    ptr = dev.ctypes.data_as(C.POINTER(C.c_int32))
    assert L.mlb_pool_new(b"nowhere.bin", ptr, 0, 4, 0, None, C.byref(h)) == api.MLB_E_INVALID
    assert L.mlb_pool_new(b"nowhere.bin", ptr, 2, 4, 0, None, C.byref(h)) == api.MLB_E_INVALID      # negative device
    assert L.mlb_pool_new(b"nowhere.bin", ptr, 1, 0, 0, None, C.byref(h)) == api.MLB_E_INVALID      # empty batch
    assert L.mlb_pool_new(None, ptr, 1, 4, 0, None, C.byref(h)) == api.MLB_E_INVALID
    assert not h


def test_fp8_tensors_in_the_model_file(api, tmp_path):
    """Offline FP8: the converter's e4m3 encoder is the hardware rounding (checked against torch's cast on a
    sweep including subnormals, ties and saturation), a float8_e4m3 file holds codes and per-row scales for the
    matrices (bf16 for the per-layer embedding, float32 for the gains), both readers return code * scale, the
    C parser accepts the file, and the file is about a quarter of the float32 one."""
    import torch
    from mini_llm_cuda_b200 import model_file as mf
    from oracle.model_bin import read_model_bin as oracle_read
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(50000).astype(np.float32) * s for s in (1e-3, 0.02, 1.0, 60.0, 300.0)] +
                       [np.array([0, -0.0, 448, -448, 500, -1e9, 2 ** -9, 2 ** -10, 1.5 * 2 ** -9, 2.5 * 2 ** -9, 447.9, 464,
                                  479.9, 15.5 * 2 ** -9, 2 ** -6, 0.99 * 2 ** -6], dtype=np.float32)])
    ref = torch.from_numpy(np.clip(x, -448, 448)).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(mf._to_e4m3_bits(x), ref)
    spec = mf.ModelSpec(dim=128, layers=2, heads=2, head_dim=64, ffn_dim=256, vocab=512, max_context=64, ple_dim=32,
                        layer_types=mf.periodic_layer_types(2, 2), weight_dtype="float8_e4m3", kv_dtype="bfloat16")
    w = mf.synth_weights(spec, seed=3)
    p32, p8 = os.path.join(str(tmp_path), "f32.bin"), os.path.join(str(tmp_path), "fp8.bin")
    mf.write_model_bin(p32, spec, w)
    mf.write_model_bin(p8, spec, w, file_dtype="float8_e4m3")
    assert os.path.getsize(p8) < 0.3 * os.path.getsize(p32)
    header, back = mf.read_model_bin(p8)
    assert header["transformerBlocks"][0]["queryWeights"]["dtype"] == "float8_e4m3"
    assert header["transformerBlocks"][0]["rmsGamma"]["dtype"] == "float32"
    assert {e["name"]: e["dtype"] for e in header["ext"]}["pleTable"] == "bfloat16"
    q = w["blocks"][0]["queryWeights"]
    codes, scale = mf.quantize_fp8_rows(q)
    want = mf._e4m3_values()[codes] * scale[:, None]
    assert np.array_equal(back["blocks"][0]["queryWeights"], want)
    assert np.abs(want - q).max() <= np.abs(q).max() / 16            # 3 mantissa bits
    assert np.array_equal(oracle_read(p8)["blocks"][0]["queryWeights"], want)
    cfg, n_params = api.inspect_file(p8)
    cfg32, n32 = api.inspect_file(p32)
    assert n_params == n32 and cfg.weight_dtype == api.DT_FP8
    # the converter: float32 file in, FP8 file out by default when the device type is FP8
    dst = os.path.join(str(tmp_path), "conv.bin")
    spec2 = mf.convert_model_bin(p32, dst, weight_dtype="float8_e4m3")
    assert spec2.weight_dtype == "float8_e4m3" and os.path.getsize(dst) == os.path.getsize(p8)
    # a truncated FP8 tensor is refused like any other
    raw = open(p8, "rb").read()
    short = os.path.join(str(tmp_path), "short.bin")
    open(short, "wb").write(raw[:len(raw) - 64])
    with pytest.raises(api.MlbError):
        api.inspect_file(short)
