"""Generates tests/golden/wire_golden.json from the REFERENCE's own codecs.

Run where the reference tree is mounted:

    make -C oracle reference REFERENCE=<path of the reference tree>
    python tests/golden/make_wire_golden.py

It drives the reference's src/protocol.c (compiled unchanged into oracle/_ref/libfgref.so)
over the output messages -- config, result, partial, history -- and the split-head layout,
and records every input with the bytes or the status the reference produced.  The fixture
travels with the repository; the reference does not.
"""
from __future__ import annotations

import ctypes
import json
import struct
import sys
from ctypes import POINTER, Structure, byref, c_bool, c_float, c_int, c_uint8, c_uint32, c_uint64, c_void_p
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
import oracle  # noqa: E402


class Sampler(Structure):
    _fields_ = [("temperature", c_float), ("top_p", c_float), ("top_k", c_uint32), ("presence_penalty", c_float),
                ("frequency_penalty", c_float), ("repetition_penalty", c_float), ("min_p", c_float),
                ("seed", c_uint64)]


class Config(Structure):
    _fields_ = [("source_rank", c_uint8), ("destination_rank", c_uint8), ("flags", c_uint8),
                ("session_slot", c_uint8), ("token_index", c_uint32), ("sampler", Sampler), ("uniform", c_float)]


class Result(Structure):
    _fields_ = [("source_rank", c_uint8), ("destination_rank", c_uint8), ("token_index", c_uint32),
                ("token", c_uint32), ("logit", c_float)]


class Partial(Structure):
    _fields_ = [("token_index", c_uint32), ("value", c_float), ("id", c_uint32)]


class History(Structure):
    _fields_ = [("tokens", POINTER(c_uint32)), ("count", c_uint32), ("session_slot", c_uint8)]


def f32(bits: int) -> float:
    return struct.unpack("<f", struct.pack("<I", bits))[0]


def bits_of(value: float) -> int:
    return struct.unpack("<I", struct.pack("<f", value))[0]


SAMPLERS = [
    dict(temperature=1.0, top_p=0.95, top_k=20, presence_penalty=0.0, frequency_penalty=0.0,
         repetition_penalty=1.0, min_p=0.0),
    dict(temperature=0.7, top_p=0.8, top_k=20, presence_penalty=1.5, frequency_penalty=0.0,
         repetition_penalty=1.0, min_p=0.0),
    dict(temperature=0.0, top_p=1.0, top_k=1, presence_penalty=0.0, frequency_penalty=0.0,
         repetition_penalty=1.0, min_p=0.0),
    dict(temperature=0.0, top_p=0.0, top_k=0, presence_penalty=0.0, frequency_penalty=0.0,
         repetition_penalty=0.0, min_p=0.0),  # all zero: "unset", let through
    dict(temperature=1.0, top_p=0.95, top_k=65, presence_penalty=0.0, frequency_penalty=0.0,
         repetition_penalty=1.0, min_p=0.0),  # invalid
    dict(temperature=1.0, top_p=0.95, top_k=50, presence_penalty=-2.0, frequency_penalty=2.0,
         repetition_penalty=1.05, min_p=0.0),
    dict(temperature=1.0, top_p=0.95, top_k=50, presence_penalty=0.0, frequency_penalty=0.0,
         repetition_penalty=1.0, min_p=0.1),  # invalid
]


def main() -> None:
    lib = oracle.load("reference")
    E = POINTER(oracle.OracleError)
    lib.fg_output_config_encode.restype = c_int
    lib.fg_output_config_encode.argtypes = [c_void_p, POINTER(Config), E]
    lib.fg_output_config_decode.restype = c_int
    lib.fg_output_config_decode.argtypes = [POINTER(Config), c_void_p, c_uint32, E]
    lib.fg_output_result_encode.restype = c_int
    lib.fg_output_result_encode.argtypes = [c_void_p, POINTER(Result), E]
    lib.fg_output_result_decode.restype = c_int
    lib.fg_output_result_decode.argtypes = [POINTER(Result), c_void_p, c_uint32, E]
    lib.fg_output_partial_encode.restype = c_int
    lib.fg_output_partial_encode.argtypes = [c_void_p, POINTER(Partial), E]
    lib.fg_output_partial_decode.restype = c_int
    lib.fg_output_partial_decode.argtypes = [POINTER(Partial), c_void_p, c_uint32, E]
    lib.fg_output_history_encode.restype = c_int
    lib.fg_output_history_encode.argtypes = [c_void_p, c_uint32, POINTER(c_uint32), POINTER(History), E]
    lib.fg_output_history_decode.restype = c_int
    lib.fg_output_history_decode.argtypes = [POINTER(History), c_void_p, c_uint32, c_void_p, c_uint32, E]
    lib.fg_output_split_way_for_rank.restype = c_bool
    lib.fg_output_split_way_for_rank.argtypes = [c_uint32, c_uint32, POINTER(c_uint32)]
    lib.fg_output_split_rank.restype = c_uint32
    lib.fg_output_split_rank.argtypes = [c_uint32, c_uint32]
    lib.fg_output_split_span.restype = None
    lib.fg_output_split_span.argtypes = [c_uint32, c_uint32, POINTER(c_uint32), POINTER(c_uint32)]

    out: dict = {"generator": "tests/golden/make_wire_golden.py", "source": "reference src/protocol.c"}

    # ---- config: encode every combination of a few routes, flags, samplers and draws ----
    cases = []
    for sampler in SAMPLERS:
        for source, destination, flags, slot, uniform_bits in [
                (0, 4, 0, 0, bits_of(0.25)), (7, 4, 1, 1, bits_of(0.0)), (3, 4, 3, 0, 0x3f7fffff),
                (8, 4, 0, 0, bits_of(0.5)), (0, 5, 0, 0, bits_of(0.5)), (0, 4, 0, 2, bits_of(0.5)),
                (0, 4, 0, 0, bits_of(1.0)), (0, 4, 0, 0, 0x7fc00000), (0, 4, 0, 0, bits_of(-0.0)),
                (0, 4, 0, 0, bits_of(-1e-9))]:
            config = Config(source, destination, flags, slot, 123456789, Sampler(seed=77, **sampler),
                            f32(uniform_bits))
            buffer = (c_uint8 * 40)()
            err = oracle.OracleError()
            status = lib.fg_output_config_encode(buffer, byref(config), byref(err))
            cases.append({"source": source, "destination": destination, "flags": flags, "slot": slot,
                          "token_index": 123456789, "sampler": sampler, "uniform_bits": uniform_bits,
                          "status": status, "bytes": bytes(buffer).hex() if status == 0 else None})
    out["config_encode"] = cases

    # ---- config: decode good bytes, then every single-byte corruption class ----
    good = Config(1, 4, 1, 1, 42, Sampler(seed=0, **SAMPLERS[1]), 0.75)
    buffer = (c_uint8 * 40)()
    assert lib.fg_output_config_encode(buffer, byref(good), byref(oracle.OracleError())) == 0
    base = bytes(buffer)
    decodes = []
    mutations = [(None, None, 40)] + [(i, v, 40) for i, v in [(0, 8), (1, 3), (2, 2), (2, 4), (2, 3), (3, 2),
                                                               (16, 0xff), (20, 0x7f), (8, 0x7f), (39, 1)]]
    mutations += [(None, None, 39), (None, None, 41), (None, None, 0)]
    for index, value, size in mutations:
        data = bytearray(base)
        if index is not None:
            data[index] = value
        data = bytes(data[:size]) if size <= 40 else bytes(data) + b"\0"
        raw = (c_uint8 * max(len(data), 1))(*data)
        decoded = Config()
        status = lib.fg_output_config_decode(byref(decoded), raw, len(data), byref(oracle.OracleError()))
        entry = {"bytes": data.hex(), "status": status}
        if status == 0:
            entry["fields"] = {"source": decoded.source_rank, "destination": decoded.destination_rank,
                               "flags": decoded.flags, "slot": decoded.session_slot,
                               "token_index": decoded.token_index,
                               "uniform_bits": bits_of(decoded.uniform),
                               "sampler_bits": [bits_of(decoded.sampler.temperature), bits_of(decoded.sampler.top_p),
                                                decoded.sampler.top_k, bits_of(decoded.sampler.presence_penalty),
                                                bits_of(decoded.sampler.frequency_penalty),
                                                bits_of(decoded.sampler.repetition_penalty),
                                                bits_of(decoded.sampler.min_p)]}
        decodes.append(entry)
    out["config_decode"] = decodes

    # ---- result ----
    cases = []
    for source, destination, token, logit_bits in [(4, 0, 0, bits_of(1.5)), (4, 7, 248319, bits_of(-3.25)),
                                                   (4, 8, 5, bits_of(0.0)), (3, 0, 5, bits_of(0.0)),
                                                   (4, 0, 248320, bits_of(0.0)), (4, 0, 5, 0x7f800000),
                                                   (4, 0, 5, 0xffc00000), (4, 2, 151935, 0x80000000)]:
        result = Result(source, destination, 99, token, f32(logit_bits))
        buffer = (c_uint8 * 16)()
        status = lib.fg_output_result_encode(buffer, byref(result), byref(oracle.OracleError()))
        entry = {"source": source, "destination": destination, "token_index": 99, "token": token,
                 "logit_bits": logit_bits, "status": status, "bytes": bytes(buffer).hex() if status == 0 else None}
        cases.append(entry)
    out["result_encode"] = cases
    decodes = []
    good = bytes.fromhex(cases[0]["bytes"])
    for index, value, size in [(None, None, 16), (2, 1, 16), (3, 9, 16), (0, 0, 16), (1, 200, 16), (8, 0xff, 16),
                               (12, 0x7f, 16), (None, None, 15), (None, None, 17)]:
        data = bytearray(good)
        if index is not None:
            data[index] = value
        data = bytes(data[:size]) if size <= 16 else bytes(data) + b"\0"
        raw = (c_uint8 * len(data))(*data)
        decoded = Result()
        status = lib.fg_output_result_decode(byref(decoded), raw, len(data), byref(oracle.OracleError()))
        entry = {"bytes": data.hex(), "status": status}
        if status == 0:
            entry["fields"] = [decoded.source_rank, decoded.destination_rank, decoded.token_index, decoded.token,
                               bits_of(decoded.logit)]
        decodes.append(entry)
    out["result_decode"] = decodes

    # ---- partial ----
    cases = []
    for token_index, value_bits, ident in [(7, bits_of(12.5), 140047), (0, bits_of(-0.0), 0),
                                           (2**32 - 1, bits_of(1e30), 248319), (1, 0x7f800000, 3),
                                           (1, 0x7fc00001, 3), (1, bits_of(1.0), 248320)]:
        partial = Partial(token_index, f32(value_bits), ident)
        buffer = (c_uint8 * 12)()
        status = lib.fg_output_partial_encode(buffer, byref(partial), byref(oracle.OracleError()))
        cases.append({"token_index": token_index, "value_bits": value_bits, "id": ident, "status": status,
                      "bytes": bytes(buffer).hex() if status == 0 else None})
    out["partial_encode"] = cases
    decodes = []
    good = bytes.fromhex(cases[0]["bytes"])
    for data in [good, good[:11], good + b"\0", bytes([0, 0, 0, 1, 0x7f, 0x80, 0, 0, 0, 0, 0, 1]),
                 bytes([0, 0, 0, 1, 0x3f, 0x80, 0, 0, 0, 3, 0xca, 0x00])]:
        raw = (c_uint8 * len(data))(*data)
        decoded = Partial()
        status = lib.fg_output_partial_decode(byref(decoded), raw, len(data), byref(oracle.OracleError()))
        entry = {"bytes": data.hex(), "status": status}
        if status == 0:
            entry["fields"] = [decoded.token_index, bits_of(decoded.value), decoded.id]
        decodes.append(entry)
    out["partial_decode"] = decodes

    # ---- history ----
    cases = []
    for tokens, slot, capacity in [([], 0, 8), ([1, 2, 3], 1, 64), ([248319, 0, 77, 77], 0, 24), ([5], 2, 64),
                                   ([248320], 0, 64), ([1, 2, 3], 0, 19), ([9] * 1000, 1, 8 + 4000)]:
        array = (c_uint32 * max(len(tokens), 1))(*tokens)
        history = History(ctypes.cast(array, POINTER(c_uint32)) if tokens else None, len(tokens), slot)
        buffer = (c_uint8 * max(capacity, 1))()
        used = c_uint32(0)
        status = lib.fg_output_history_encode(buffer, capacity, byref(used), byref(history),
                                              byref(oracle.OracleError()))
        cases.append({"tokens": tokens if len(tokens) < 20 else {"repeat": tokens[0], "count": len(tokens)},
                      "slot": slot, "capacity": capacity, "status": status,
                      "bytes": bytes(buffer[:used.value]).hex() if status == 0 else None})
    out["history_encode"] = cases
    decodes = []
    good = bytes.fromhex(cases[2]["bytes"])
    for data, capacity in [(good, 16), (good, 3), (good[:-1], 16), (good + b"\0\0\0\0", 16),
                           (good[:4] + bytes([2]) + good[5:], 16), (good[:5] + bytes([1]) + good[6:], 16),
                           (good[:8] + bytes([0, 3, 0xca, 0]) + good[12:], 16), (good[:7], 16),
                           (bytes.fromhex(cases[0]["bytes"]), 0)]:
        raw = (c_uint8 * max(len(data), 1))(*data)
        storage = (c_uint32 * max(capacity, 1))()
        decoded = History()
        status = lib.fg_output_history_decode(byref(decoded), storage, capacity, raw, len(data),
                                              byref(oracle.OracleError()))
        entry = {"bytes": data.hex(), "capacity": capacity, "status": status}
        if status == 0:
            entry["tokens"] = [storage[i] for i in range(decoded.count)]
            entry["slot"] = decoded.session_slot
        decodes.append(entry)
    out["history_decode"] = decodes

    # ---- split layout ----
    layout = []
    for ways in (1, 2, 3, 4, 5):
        for index in range(9):
            way = c_uint32(0xdead)
            found = lib.fg_output_split_way_for_rank(ways, index, byref(way))
            first, rows = c_uint32(1), c_uint32(1)
            lib.fg_output_split_span(ways, index, byref(first), byref(rows))
            layout.append({"ways": ways, "index": index, "way_for_rank": [bool(found), way.value if found else None],
                           "rank_of_way": lib.fg_output_split_rank(ways, index),
                           "span": [first.value, rows.value]})
    out["split_layout"] = layout

    path = Path(__file__).resolve().parent / "wire_golden.json"
    path.write_text(json.dumps(out, indent=1) + "\n")
    print(f"wrote {path} ({path.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
