"""`.litertlm` container: reader against the reference's binary fixture, writer round trips.

Reference: schema/core/litertlm_export.cc:126-173 (layout), litertlm_read.cc:38-109 (header
checks), litertlm_read_test.cc:157-171 (HF tokenizer section inflates to tokenizer.json),
schema/testdata/llm_metadata.pb (LlmMetadata wire bytes).
"""
import hashlib
import json
import os
import struct

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
# a checkout of the reference, when one is mounted (LITERT_LM_REFERENCE); the committed golden header is used otherwise
REF_FIXTURE = os.path.join(os.environ.get("LITERT_LM_REFERENCE", os.path.join(os.sep, "root", "reference")),
                           "schema", "testdata", "test_hf_tokenizer.litertlm")


@pytest.fixture(scope="module")
def golden():
    with open(os.path.join(GOLDEN, "litertlm_fixture.json")) as f:
        return json.load(f)


def test_decode_reference_header_bytes(mio, golden):
    """The flatbuffer header bytes of the reference's fixture decode to its metadata."""
    fb = bytes.fromhex(golden["header_flatbuffer_hex"])
    system, sections = mio.decode_header(fb)
    assert [(k, v) for k, v, _ in system] == [("arch", "all"), ("version", "0.1")]
    assert len(sections) == 1
    s = sections[0]
    assert s.data_type == mio.SECTION_HF_TOKENIZER_ZLIB
    assert s.begin == 16384 and s.end == golden["sections"][0]["end"] == 609288
    assert s.begin % mio.BLOCK == 0


@pytest.mark.skipif(not os.path.exists(REF_FIXTURE), reason="reference checkout not present")
def test_reference_fixture_file(mio, golden):
    data = open(REF_FIXTURE, "rb").read()
    lf = mio.read_litertlm(data)
    assert len(data) == golden["file_size"] == 622592
    assert lf.version[0] == 1 and lf.header_end == golden["header_end"] == 240
    sec = lf.sections[0]
    tok = mio.read_hf_tokenizer_section(data[sec.begin:sec.end])
    assert len(tok) == golden["tokenizer_json_size"] == 2104556
    assert hashlib.sha256(tok).hexdigest() == golden["tokenizer_json_sha256"]


def test_llm_metadata_wire_bytes(mio, golden):
    mine = mio.llm_metadata_proto(0, start_token_str="<bos>", stop_token_strs=["<eos>", "<end_of_turn>"])
    assert mine.hex() == golden["llm_metadata_pb_hex"]


def test_header_reader_checks(mio):
    with pytest.raises(ValueError):
        mio.read_litertlm(b"NOTLITER" + b"\0" * 64)
    bad_major = bytearray(mio.write_litertlm([(mio.SECTION_GENERIC, b"abc", [])]))
    struct.pack_into("<I", bad_major, 8, 2)
    with pytest.raises(NotImplementedError):
        mio.read_litertlm(bytes(bad_major))
    with pytest.raises(ValueError):
        mio.write_litertlm([])


def test_writer_round_trip_typed_metadata(mio):
    """The cases of litertlm_header_test.cc:75-183: typed system metadata and two sections."""
    system = [("str", "hello"), ("i32", 2048), ("f32", 1.5), ("flag", True), ("u64", (mio.VD_UINT64, 2 ** 40)),
              ("i64", -2 ** 40), ("u8", (mio.VD_UINT8, 200))]
    payload_a, payload_b = os.urandom(20000), b"\x01\x02\x03"
    img = mio.write_litertlm([(mio.SECTION_TFLITE, payload_a, [("model_type", "tf_lite_prefill_decode"), ("q", True)]),
                              (mio.SECTION_GENERIC, payload_b, [])], system_kv=system)
    assert img[:8] == b"LITERTLM" and struct.unpack_from("<III", img, 8) == (1, 1, 0)
    lf = mio.read_litertlm(img)
    got = {k: v for k, v, _ in lf.system}
    assert got["str"] == "hello" and got["i32"] == 2048 and got["f32"] == 1.5 and got["flag"] is True
    assert got["u64"] == 2 ** 40 and got["i64"] == -2 ** 40 and got["u8"] == 200
    a, b = lf.sections
    assert (a.begin, a.end) == (16384, 16384 + 20000) and b.begin == 49152       # next 16 KiB boundary
    assert img[a.begin:a.end] == payload_a and img[b.begin:b.end] == payload_b
    assert [(k, v) for k, v, _ in a.items] == [("model_type", "tf_lite_prefill_decode"), ("q", True)]
    assert len(img) % mio.BLOCK == 0


def test_hf_tokenizer_section_round_trip(mio):
    blob = json.dumps({"x": list(range(1000))}).encode()
    assert mio.read_hf_tokenizer_section(mio.hf_tokenizer_section(blob)) == blob


def test_model_export_round_trip(mio, models):
    cfg, rec, img = models("tiny")
    assert mio.find_weights_record(img) == rec
    cfg2, tensors = mio.parse_weights_record(rec)
    assert (cfg2.n_layers, cfg2.d_model, cfg2.head_dim, cfg2.buckets) == (cfg.n_layers, cfg.d_model, cfg.head_dim, cfg.buckets)
    assert tensors["embed.q"].shape == (cfg.vocab, cfg.d_model // 2)
    assert tensors["L1.wdown.q"].shape == (cfg.d_model, cfg.ffn // 2)
    lf = mio.read_litertlm(img)
    assert [s.data_type for s in lf.sections] == [mio.SECTION_LLM_METADATA, mio.SECTION_GENERIC]


def test_weight_generation_is_seeded(mio):
    a = mio.build_weights_record(mio.config_tiny(seed=5))
    b = mio.build_weights_record(mio.config_tiny(seed=5))
    c = mio.build_weights_record(mio.config_tiny(seed=6))
    assert a == b and a != c
