"""The output-message codecs and the logit-dump reader of include/fg_output_wire.h against
tests/golden/wire_golden.json, which tests/golden/make_wire_golden.py recorded from the
reference's own src/protocol.c: every encode must give the reference's bytes or its status,
every decode the reference's fields or its status (tests/test_core.c:940-976 and
tests/test_fabric.c of the reference check the same codecs by round trip)."""
import ctypes
import json
import struct
from ctypes import POINTER, Structure, byref, c_bool, c_char_p, c_float, c_int, c_uint8, c_uint32, c_void_p
from pathlib import Path

import numpy as np
import pytest

import flash_gordon_b200 as fg
from flash_gordon_b200 import FG_OK, FgError, SamplerConfig

GOLDEN = json.loads((Path(__file__).resolve().parent / "golden" / "wire_golden.json").read_text())


class Config(Structure):
    _fields_ = [("source_rank", c_uint8), ("destination_rank", c_uint8), ("flags", c_uint8),
                ("session_slot", c_uint8), ("token_index", c_uint32), ("sampler", SamplerConfig),
                ("uniform", c_float)]


class Result(Structure):
    _fields_ = [("source_rank", c_uint8), ("destination_rank", c_uint8), ("token_index", c_uint32),
                ("token", c_uint32), ("logit", c_float)]


class Partial(Structure):
    _fields_ = [("token_index", c_uint32), ("value", c_float), ("id", c_uint32)]


class History(Structure):
    _fields_ = [("tokens", POINTER(c_uint32)), ("count", c_uint32), ("session_slot", c_uint8)]


class Limits(Structure):
    _fields_ = [("rank_count", c_uint32), ("output_rank", c_uint32), ("session_slots", c_uint32),
                ("vocab", c_uint32)]


def f32(bits):
    return struct.unpack("<f", struct.pack("<I", bits))[0]


def bits_of(value):
    return struct.unpack("<I", struct.pack("<f", value))[0]


@pytest.fixture(scope="module")
def wire(library):
    lib = library
    E = POINTER(FgError)
    for name, argtypes in {
        "fg_output_config_encode": [c_void_p, POINTER(Config), E],
        "fg_output_config_decode": [POINTER(Config), c_void_p, c_uint32, E],
        "fg_output_result_encode": [c_void_p, POINTER(Result), E],
        "fg_output_result_decode": [POINTER(Result), c_void_p, c_uint32, E],
        "fg_output_partial_encode": [c_void_p, POINTER(Partial), E],
        "fg_output_partial_decode": [POINTER(Partial), c_void_p, c_uint32, E],
        "fg_output_history_encode": [c_void_p, c_uint32, POINTER(c_uint32), POINTER(History), E],
        "fg_output_history_decode": [POINTER(History), c_void_p, c_uint32, c_void_p, c_uint32, E],
        "fg_output_result_encode_with": [POINTER(Limits), c_void_p, POINTER(Result), E],
        "fg_output_result_decode_with": [POINTER(Limits), POINTER(Result), c_void_p, c_uint32, E],
        "fg_output_history_encode_with": [POINTER(Limits), c_void_p, c_uint32, POINTER(c_uint32), POINTER(History), E],
        "fg_logit_dump_read": [c_char_p, c_void_p, c_uint32, POINTER(c_uint32), c_bool, E],
        "fg_logit_dump_write": [c_char_p, c_void_p, c_uint32, E],
    }.items():
        getattr(lib, name).restype = c_int
        getattr(lib, name).argtypes = argtypes
    lib.fg_output_split_way_for_rank.restype = c_bool
    lib.fg_output_split_way_for_rank.argtypes = [c_uint32, c_uint32, POINTER(c_uint32)]
    lib.fg_output_split_rank.restype = c_uint32
    lib.fg_output_split_rank.argtypes = [c_uint32, c_uint32]
    lib.fg_output_split_span.restype = None
    lib.fg_output_split_span.argtypes = [c_uint32, c_uint32, POINTER(c_uint32), POINTER(c_uint32)]
    lib.fg_wire_limits_reference.restype = Limits
    lib.fg_wire_limits_reference.argtypes = []
    return lib


def raw_buffer(data: bytes):
    return (c_uint8 * max(len(data), 1))(*data)


def test_struct_layouts_are_the_reference_s():
    assert ctypes.sizeof(Config) == 56 and Config.sampler.offset == 8 and Config.uniform.offset == 48
    assert ctypes.sizeof(Result) == 16 and ctypes.sizeof(Partial) == 12


def test_config_codec_matches_the_reference(wire):
    for case in GOLDEN["config_encode"]:
        s = case["sampler"]
        sampler = SamplerConfig(s["temperature"], s["top_p"], s["top_k"], s["presence_penalty"],
                                s["frequency_penalty"], s["repetition_penalty"], s["min_p"])
        sampler.seed = 77
        config = Config(case["source"], case["destination"], case["flags"], case["slot"], case["token_index"],
                        sampler, f32(case["uniform_bits"]))
        buffer = (c_uint8 * 40)(*([0xEE] * 40))
        status = wire.fg_output_config_encode(buffer, byref(config), byref(FgError()))
        assert status == case["status"], case
        if status == FG_OK:
            assert bytes(buffer).hex() == case["bytes"], case
    for case in GOLDEN["config_decode"]:
        data = bytes.fromhex(case["bytes"])
        decoded = Config()
        status = wire.fg_output_config_decode(byref(decoded), raw_buffer(data), len(data), byref(FgError()))
        assert status == case["status"], case
        if status == FG_OK:
            f = case["fields"]
            got = [bits_of(decoded.sampler.temperature), bits_of(decoded.sampler.top_p), decoded.sampler.top_k,
                   bits_of(decoded.sampler.presence_penalty), bits_of(decoded.sampler.frequency_penalty),
                   bits_of(decoded.sampler.repetition_penalty), bits_of(decoded.sampler.min_p)]
            assert (decoded.source_rank, decoded.destination_rank, decoded.flags, decoded.session_slot,
                    decoded.token_index, bits_of(decoded.uniform)) == (
                f["source"], f["destination"], f["flags"], f["slot"], f["token_index"], f["uniform_bits"])
            assert got == f["sampler_bits"]


def test_result_and_partial_codecs_match_the_reference(wire):
    for case in GOLDEN["result_encode"]:
        result = Result(case["source"], case["destination"], case["token_index"], case["token"],
                        f32(case["logit_bits"]))
        buffer = (c_uint8 * 16)(*([0xEE] * 16))
        status = wire.fg_output_result_encode(buffer, byref(result), byref(FgError()))
        assert status == case["status"], case
        if status == FG_OK:
            assert bytes(buffer).hex() == case["bytes"]
    for case in GOLDEN["result_decode"]:
        data = bytes.fromhex(case["bytes"])
        decoded = Result()
        status = wire.fg_output_result_decode(byref(decoded), raw_buffer(data), len(data), byref(FgError()))
        assert status == case["status"], case
        if status == FG_OK:
            assert [decoded.source_rank, decoded.destination_rank, decoded.token_index, decoded.token,
                    bits_of(decoded.logit)] == case["fields"]
    for case in GOLDEN["partial_encode"]:
        partial = Partial(case["token_index"], f32(case["value_bits"]), case["id"])
        buffer = (c_uint8 * 12)(*([0xEE] * 12))
        status = wire.fg_output_partial_encode(buffer, byref(partial), byref(FgError()))
        assert status == case["status"], case
        if status == FG_OK:
            assert bytes(buffer).hex() == case["bytes"]
    for case in GOLDEN["partial_decode"]:
        data = bytes.fromhex(case["bytes"])
        decoded = Partial()
        status = wire.fg_output_partial_decode(byref(decoded), raw_buffer(data), len(data), byref(FgError()))
        assert status == case["status"], case
        if status == FG_OK:
            assert [decoded.token_index, bits_of(decoded.value), decoded.id] == case["fields"]


def test_history_codec_matches_the_reference(wire):
    for case in GOLDEN["history_encode"]:
        tokens = case["tokens"]
        if isinstance(tokens, dict):
            tokens = [tokens["repeat"]] * tokens["count"]
        array = (c_uint32 * max(len(tokens), 1))(*tokens)
        history = History(ctypes.cast(array, POINTER(c_uint32)) if tokens else None, len(tokens), case["slot"])
        buffer = (c_uint8 * max(case["capacity"], 1))()
        used = c_uint32(0)
        status = wire.fg_output_history_encode(buffer, case["capacity"], byref(used), byref(history),
                                               byref(FgError()))
        assert status == case["status"], case
        if status == FG_OK:
            assert bytes(buffer[:used.value]).hex() == case["bytes"]
    for case in GOLDEN["history_decode"]:
        data = bytes.fromhex(case["bytes"])
        storage = (c_uint32 * max(case["capacity"], 1))()
        decoded = History()
        status = wire.fg_output_history_decode(byref(decoded), storage, case["capacity"], raw_buffer(data),
                                               len(data), byref(FgError()))
        assert status == case["status"], case
        if status == FG_OK:
            assert [storage[i] for i in range(decoded.count)] == case["tokens"]
            assert decoded.session_slot == case["slot"]


def test_split_layout_matches_the_reference(wire):
    for case in GOLDEN["split_layout"]:
        way = c_uint32(0xdead)
        found = wire.fg_output_split_way_for_rank(case["ways"], case["index"], byref(way))
        assert [bool(found), way.value if found else None] == case["way_for_rank"], case
        assert wire.fg_output_split_rank(case["ways"], case["index"]) == case["rank_of_way"], case
        first, rows = c_uint32(1), c_uint32(1)
        wire.fg_output_split_span(case["ways"], case["index"], byref(first), byref(rows))
        assert [first.value, rows.value] == case["span"], case


def test_other_limits_for_another_vocabulary(wire):
    """The *_with variants: the benchmark's 151,936-token vocabulary on a 16-rank layout."""
    limits = Limits(16, 9, 64, 151_936)
    result = Result(9, 15, 1, 151_935, 2.5)
    buffer = (c_uint8 * 16)()
    assert wire.fg_output_result_encode_with(byref(limits), buffer, byref(result), byref(FgError())) == FG_OK
    decoded = Result()
    assert wire.fg_output_result_decode_with(byref(limits), byref(decoded), buffer, 16, byref(FgError())) == FG_OK
    assert (decoded.token, decoded.destination_rank) == (151_935, 15)
    result.token = 151_936
    assert wire.fg_output_result_encode_with(byref(limits), buffer, byref(result), byref(FgError())) != FG_OK
    reference = wire.fg_wire_limits_reference()
    assert (reference.rank_count, reference.output_rank, reference.session_slots, reference.vocab) == (8, 4, 2, 248_320)
    tokens = (c_uint32 * 2)(151_935, 3)
    history = History(ctypes.cast(tokens, POINTER(c_uint32)), 2, 63)
    out, used = (c_uint8 * 16)(), c_uint32(0)
    assert wire.fg_output_history_encode_with(byref(limits), out, 16, byref(used), byref(history),
                                              byref(FgError())) == FG_OK and used.value == 16


def test_logit_dump_round_trip_and_refusals(wire, tmp_path):
    values = np.random.default_rng(4).standard_normal(1000).astype(np.float32)
    path = tmp_path / "0000.fgl"
    encoded = str(path).encode()
    assert wire.fg_logit_dump_write(encoded, values.ctypes.data_as(c_void_p), 1000, byref(FgError())) == FG_OK
    raw = path.read_bytes()
    # the layout the reference writes (src/output.c:580-584) and its tool reads back
    assert raw[:8] == b"FGLOG01\n" and struct.unpack("<I", raw[8:12])[0] == 1000 and len(raw) == 12 + 4000
    assert np.array_equal(np.frombuffer(raw[12:], dtype="<f4"), values)
    back = np.zeros(1000, dtype=np.float32)
    count = c_uint32(0)
    assert wire.fg_logit_dump_read(encoded, back.ctypes.data_as(c_void_p), 1000, byref(count), True,
                                   byref(FgError())) == FG_OK
    assert count.value == 1000 and np.array_equal(back.view(np.uint32), values.view(np.uint32))
    assert wire.fg_logit_dump_read(encoded, None, 0, byref(count), True, byref(FgError())) == FG_OK  # size only
    assert wire.fg_logit_dump_read(encoded, back.ctypes.data_as(c_void_p), 999, byref(count), True,
                                   byref(FgError())) == fg.FG_ERR_LIMIT
    path.write_bytes(raw[:-1])
    assert wire.fg_logit_dump_read(encoded, None, 0, byref(count), True, byref(FgError())) == fg.FG_ERR_FORMAT
    path.write_bytes(b"FGLOG02\n" + raw[8:])
    assert wire.fg_logit_dump_read(encoded, None, 0, byref(count), True, byref(FgError())) == fg.FG_ERR_FORMAT
    bad = values.copy()
    bad[17] = np.nan
    path.write_bytes(raw[:12] + bad.tobytes())
    assert wire.fg_logit_dump_read(encoded, back.ctypes.data_as(c_void_p), 1000, byref(count), True,
                                   byref(FgError())) == fg.FG_ERR_FORMAT
    assert wire.fg_logit_dump_read(encoded, back.ctypes.data_as(c_void_p), 1000, byref(count), False,
                                   byref(FgError())) == FG_OK
    assert wire.fg_logit_dump_read(str(tmp_path / "missing.fgl").encode(), None, 0, byref(count), True,
                                   byref(FgError())) == fg.FG_ERR_IO
