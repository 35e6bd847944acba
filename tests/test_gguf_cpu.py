"""The GGUF reader against the reference's own test cases (crates/xabe-gguf/src/file.rs:585-752,
crates/xabe-gguf/src/types.rs:135-181), through the C ABI of libxabe_gguf.so.  CPU only."""
import os
import struct

import numpy as np
import pytest

from gguf_builder import Builder


def _err(data: bytes) -> str:
    from llmxabe_b200.gguf import GgufError, GgufFile
    with pytest.raises(GgufError) as e:
        GgufFile.from_bytes(data)
    return e.value.kind


def test_block_sizes_match_ggml_type_traits():
    """types.rs `block_sizes_match_ggml_type_traits`, `bytes_for_elements_rejects_partial_blocks`,
    `try_from_round_trips_ggml_type_ids`."""
    from llmxabe_b200.gguf import GgmlType, GgufError, lib
    want = {GgmlType.F32: (1, 4), GgmlType.F16: (1, 2), GgmlType.BF16: (1, 2), GgmlType.Q4_0: (32, 18),
            GgmlType.Q8_0: (32, 34), GgmlType.Q4K: (256, 144), GgmlType.Q5K: (256, 176), GgmlType.Q6K: (256, 210)}
    for t, (block, size) in want.items():
        assert (t.block_size(), t.type_size()) == (block, size)
    assert [t.type_name() for t in (GgmlType.Q6K, GgmlType.Q8_0, GgmlType.BF16)] == ["q6_K", "q8_0", "bf16"]
    assert GgmlType.Q6K.bytes_for_elements(256) == 210 and GgmlType.Q6K.bytes_for_elements(512) == 420
    with pytest.raises(GgufError) as e:
        GgmlType.Q6K.bytes_for_elements(255)
    assert e.value.kind == "UnalignedElementCount"
    assert lib().xabe_ggml_block_size(99) == 0 and lib().xabe_ggml_type_name(99) is None
    assert sorted(int(t) for t in GgmlType) == [0, 1, 2, 8, 12, 13, 14, 30]


def test_round_trips_header_metadata_and_tensors():
    """file.rs `round_trips_header_metadata_and_tensors`, with data in the small tensor."""
    from llmxabe_b200.gguf import GgmlType, GgufFile
    norm = np.arange(2048, dtype=np.float32)
    data = (Builder()
            .kv_u32("general.alignment", 32)
            .kv_str("general.architecture", "qwen35moe")
            .kv_u32("qwen35moe.block_count", 40)
            .kv_f32("qwen35moe.attention.layer_norm_rms_epsilon", 1e-6)
            .kv_string_array("tokenizer.ggml.tokens", ["a", "b", "c"])
            .kv_array("some.array", 4, "I", [1, 2, 3, 4])
            .tensor("blk.0.attn_norm.weight", [2048], "f32", norm.tobytes())
            .tensor("blk.0.ffn_gate_exps.weight", [2048, 512, 4], "q6_K")
            .build())
    f = GgufFile.from_bytes(data)
    assert (f.version(), f.alignment(), f.n_kv(), f.n_tensors()) == (3, 32, 6, 2)
    assert f.get_u32("general.alignment") == 32
    assert f.get_str("general.architecture") == "qwen35moe"
    assert f.get_u32("qwen35moe.block_count") == 40
    assert abs(f.get_f32("qwen35moe.attention.layer_norm_rms_epsilon") - 1e-6) < 1e-12
    assert f.get_array("tokenizer.ggml.tokens") == ["a", "b", "c"]
    assert f.get_array("some.array").tolist() == [1, 2, 3, 4] and f.get_array("some.array").dtype == np.uint32
    # type mismatch -> None, not an exception or a coerced value
    assert f.get_u64("general.alignment") is None
    assert f.get_str("nonexistent.key") is None
    assert f.metadata_keys()[:2] == ["general.alignment", "general.architecture"]
    t0 = f.tensor("blk.0.attn_norm.weight")
    assert t0.dims == (2048,) and t0.ggml_type == GgmlType.F32 and t0.n_bytes == 2048 * 4
    assert np.array_equal(np.frombuffer(t0.data.tobytes(), dtype=np.float32), norm)
    t1 = f.tensor("blk.0.ffn_gate_exps.weight")
    assert t1.n_elements == 2048 * 512 * 4 and t1.n_bytes == 2048 * 512 * 4 // 256 * 210
    assert t1.offset % 32 == 0 and f.data_offset() % 32 == 0
    assert len(f.tensor_bytes("blk.0.attn_norm.weight")) == t0.n_bytes
    assert f.tensor("does.not.exist") is None and f.tensor_bytes("does.not.exist") is None
    assert [t.name for t in f.tensors()] == ["blk.0.attn_norm.weight", "blk.0.ffn_gate_exps.weight"]


def test_every_scalar_and_array_type_is_read():
    from llmxabe_b200.gguf import GgufFile
    b = Builder().kv_u64("u64", 2 ** 40).kv_bool("flag", True).kv_array("bools", 7, "b", [1, 0, 2])
    b.kv_array("f64s", 12, "d", [0.5, -2.0]).kv_array("i8s", 1, "b", [-3, 4]).kv_array("empty", 5, "i", [])
    b.kv_raw("i16", 3, struct.pack("<h", -7)).kv_str("text", "héllo ✓")
    f = GgufFile.from_bytes(b.build())
    assert f.get_u64("u64") == 2 ** 40 and f.get_bool("flag") is True
    assert f.get_array("bools").tolist() == [True, False, True]
    assert f.get_array("f64s").tolist() == [0.5, -2.0] and f.get_array("i8s").tolist() == [-3, 4]
    assert f.get_array("empty").size == 0
    assert f.get_str("text") == "héllo ✓"
    assert f.get_u32("i16") is None


def test_rejections_mirror_the_reference():
    """file.rs tests `rejects_*` and `default_alignment_is_32_when_key_absent`."""
    from llmxabe_b200.gguf import GgufFile
    ok = Builder().build()
    assert _err(b"X" + ok[1:]) == "BadMagic"
    assert _err(ok[:4] + struct.pack("<I", 2) + ok[8:]) == "UnsupportedVersion"
    full = Builder().kv_u32("general.alignment", 32).tensor("t", [32], "f32").build()
    assert _err(full[:-16]) == "TensorOutOfBounds"
    assert _err(b"GGUF") == "UnexpectedEof"
    assert _err(Builder().tensor("t", [32], "f32").build()[:-4]) == "TensorOutOfBounds"
    assert _err(Builder().tensor("t", [100], "q6_K").build()) == "UnalignedElementCount"
    assert _err(Builder().tensor("t", [2048, 0], "f32").build()) == "ZeroDimension"
    assert _err(Builder().tensor("t", [32], "f32").tensor("t", [32], "f32").build()) == "DuplicateTensor"
    assert _err(Builder().kv_u32("dup", 1).kv_u32("dup", 2).build()) == "DuplicateKey"
    assert _err(Builder().kv_u32("general.alignment", 3).build()) == "BadAlignment"
    assert GgufFile.from_bytes(Builder().tensor("t", [32], "f32").build()).alignment() == 32
    # the remaining variants of GgufError
    assert _err(Builder().kv_u64("general.alignment", 32).build()) == "BadAlignmentType"
    assert _err(Builder().kv_raw("k", 99, b"").build()) == "UnknownValueType"
    assert _err(Builder().kv_raw("k", 9, struct.pack("<iQ", 9, 0)).build()) == "NestedArray"
    assert _err(Builder().tensor("t", [2, 2, 2, 2, 2], "f32").build()) == "TooManyDimensions"
    assert _err(Builder().tensor("t", [32], "f32", type_id=99).build()) == "UnsupportedGgmlType"
    assert _err(ok[:8] + struct.pack("<q", -1) + ok[16:]) == "NegativeCount"
    assert _err(Builder().kv_raw("k", 8, struct.pack("<Q", 2) + b"\xff\xfe").build()) == "InvalidUtf8"
    assert _err(Builder().kv_raw("k", 9, struct.pack("<iQ", 4, 2 ** 60)).build()) == "UnexpectedEof"
    huge = Builder().tensor("t", [32], "f32")
    huge.infos[0] = huge.infos[0][:-8] + struct.pack("<Q", 2 ** 64 - 8)
    assert _err(huge.build()) == "OffsetOverflow"


def test_open_maps_a_file_and_views_keep_it_alive(tmp_path):
    from llmxabe_b200.gguf import GgufError, GgufFile
    payload = np.arange(64, dtype=np.float32)
    path = os.path.join(tmp_path, "tiny.gguf")
    with open(path, "wb") as fh:
        fh.write(Builder().kv_str("general.name", "tiny").tensor("w", [64], "f32", payload.tobytes()).build())
    view = GgufFile.open(path).tensor_bytes("w")  # the file object is dropped here; the view holds it
    assert np.array_equal(np.frombuffer(view.tobytes(), dtype=np.float32), payload)
    with pytest.raises(GgufError) as e:
        GgufFile.open(os.path.join(tmp_path, "missing.gguf"))
    assert e.value.kind == "Io"


def test_moe_layer_schema_names_and_shapes():
    """Role::suffix and the MoE shapes of crates/xabe-model/src/weights.rs:173-212,403-413."""
    from llmxabe_b200.gguf import GgmlType, GgufError, GgufFile
    H, F, E = 512, 256, 8

    def layer(b, l, router_type="f32", drop=None, down_dims=None):
        names = {"post_attention_norm.weight": ([H], "f32"), "ffn_gate_inp.weight": ([H, E], router_type),
                 "ffn_gate_exps.weight": ([H, F, E], "q6_K"), "ffn_up_exps.weight": ([H, F, E], "q6_K"),
                 "ffn_down_exps.weight": (down_dims or [F, H, E], "q8_0"), "ffn_gate_inp_shexp.weight": ([H], "f32"),
                 "ffn_gate_shexp.weight": ([H, F], "q8_0"), "ffn_up_shexp.weight": ([H, F], "q8_0"),
                 "ffn_down_shexp.weight": ([F, H], "q8_0")}
        for suffix, (dims, ty) in names.items():
            if suffix != drop:
                b.tensor(f"blk.{l}.{suffix}", dims, ty)
        return b

    f = GgufFile.from_bytes(layer(layer(Builder(), 0), 3, router_type="bf16").build())
    t = f.moe_layer_tensors(3, H, F, E)
    assert set(t) == {"post_norm", "router", "gate_exps", "up_exps", "down_exps", "shared_gate_inp", "shared_gate",
                      "shared_up", "shared_down"}
    assert t["router"].name == "blk.3.ffn_gate_inp.weight" and t["router"].ggml_type == GgmlType.BF16
    assert t["gate_exps"].dims == (H, F, E) and t["gate_exps"].n_bytes == H * F * E // 256 * 210
    assert t["down_exps"].ggml_type == GgmlType.Q8_0 and t["down_exps"].dims == (F, H, E)
    for kwargs, what in ((dict(drop="ffn_up_exps.weight"), "missing tensor blk.0.ffn_up_exps.weight"),
                         (dict(down_dims=[H, F, E]), "blk.0.ffn_down_exps.weight has shape")):
        g = GgufFile.from_bytes(layer(Builder(), 0, **kwargs).build())
        with pytest.raises(GgufError, match=what) as e:
            g.moe_layer_tensors(0, H, F, E)
        assert e.value.kind == "Schema"
    with pytest.raises(GgufError, match="missing tensor blk.1"):
        f.moe_layer_tensors(1, H, F, E)
