"""fg_sampler_config_from_json (include/fg_request.h) on the cases the reference's own API test
holds for its sampler fields (tests/test_api.c:1000-1064: the mapping of a full request, the
defaults, and the seven range errors), plus the texts of src/api.c:1613-1630 and malformed
bodies."""
import ctypes
from ctypes import POINTER, byref, c_char_p, c_int, c_size_t

import pytest

from flash_gordon_b200 import FG_ERR_ARGUMENT, FG_ERR_FORMAT, FG_OK, FgError, SamplerConfig


@pytest.fixture(scope="module")
def parse(library):
    fn = library.fg_sampler_config_from_json
    fn.restype = c_int
    fn.argtypes = [c_char_p, c_size_t, POINTER(SamplerConfig), POINTER(FgError)]

    def run(text: str):
        body = text.encode()
        config, err = SamplerConfig(), FgError()
        status = fn(body, len(body), byref(config), byref(err))
        return status, config, err.text()

    return run


MESSAGES = '"messages":[{"role":"user","content":"hi \\"there\\" {[,]}"}]'


def test_the_reference_s_full_request_maps_field_by_field(parse):
    status, cfg, _ = parse('{"temperature":0.5,"top_p":0.8,"top_k":20,"seed":7,"min_p":0,'
                           '"presence_penalty":1.5,"frequency_penalty":0.25,"repetition_penalty":1,' + MESSAGES + '}')
    assert status == FG_OK
    assert (cfg.temperature, cfg.top_k, cfg.seed, cfg.min_p, cfg.presence_penalty, cfg.frequency_penalty,
            cfg.repetition_penalty) == (0.5, 20, 7, 0.0, 1.5, 0.25, 1.0)
    assert cfg.top_p == ctypes.c_float(0.8).value
    status, cfg, _ = parse('{"temperature":0.7,"top_p":0.8,"top_k":20,"min_p":0,"presence_penalty":1.5,'
                           '"frequency_penalty":0,"repetition_penalty":1,' + MESSAGES + '}')
    assert status == FG_OK and cfg.temperature == ctypes.c_float(0.7).value and cfg.presence_penalty == 1.5


def test_omitted_fields_take_the_documented_defaults(parse):
    status, cfg, _ = parse('{' + MESSAGES + '}')
    assert status == FG_OK
    assert (cfg.temperature, cfg.top_k) == (1.0, 20) and cfg.top_p == ctypes.c_float(0.95).value
    assert (cfg.presence_penalty, cfg.frequency_penalty, cfg.repetition_penalty, cfg.min_p) == (0.0, 0.0, 1.0, 0.0)
    assert parse("{}")[0] == FG_OK and parse("  { }  ")[0] == FG_OK
    status, cfg, _ = parse('{"temperature":0,' + MESSAGES + '}')
    assert status == FG_OK and cfg.temperature == 0.0  # the greedy path


@pytest.mark.parametrize("field,text", [
    ('"temperature":-1', "temperature must be a finite non-negative number"),
    ('"temperature":"hot"', "temperature must be a finite non-negative number"),
    ('"temperature":1e39', "temperature must be a finite non-negative number"),
    ('"top_p":0', "top_p must be greater than 0 and at most 1"),
    ('"top_p":1.0001', "top_p must be greater than 0 and at most 1"),
    ('"top_k":65', "top_k must be an integer from 1 through 64"),
    ('"top_k":0', "top_k must be an integer from 1 through 64"),
    ('"top_k":2.5', "top_k must be an integer from 1 through 64"),
    ('"top_k":null', "top_k must be an integer from 1 through 64"),
    ('"seed":-1', "seed must be a non-negative integer"),
    ('"seed":1.5', "seed must be a non-negative integer"),
    ('"seed":9007199254740992', "seed must be a non-negative integer"),
    ('"presence_penalty":[1]', "presence_penalty must be finite"),
    ('"frequency_penalty":true', "frequency_penalty must be finite"),
    ('"repetition_penalty":{}', "repetition_penalty must be finite"),
    ('"min_p":0.1', "min_p currently supports only 0"),
    ('"presence_penalty":2.1', "invalid sampler controls"),
    ('"frequency_penalty":-2.1', "invalid sampler controls"),
    ('"repetition_penalty":0', "invalid sampler controls"),
])
def test_range_errors_carry_the_reference_s_texts(parse, field, text):
    status, _, message = parse('{' + MESSAGES + ',' + field + '}')
    assert status == FG_ERR_ARGUMENT and message == text


def test_edges_that_are_allowed(parse):
    ok = ['"top_p":1', '"top_k":64', '"top_k":1', '"top_k":6.4e1', '"seed":9007199254740991', '"presence_penalty":-2',
          '"frequency_penalty":2.0', '"repetition_penalty":1e-3', '"min_p":0.0', '"min_p":-0', '"temperature":3.4e38']
    for field in ok:
        assert parse('{' + field + '}')[0] == FG_OK, field
    # the first of two equal members counts; members nested deeper are not the request's
    status, cfg, _ = parse('{"top_k":5,"top_k":900,"nested":{"top_k":77,"temperature":-5},"list":[{"top_p":9}]}')
    assert status == FG_OK and cfg.top_k == 5 and cfg.temperature == 1.0
    # the first failing field in the reference's order is reported, wherever it stands in the body
    assert parse('{"min_p":3,"top_k":99,"temperature":-2}')[2] == "temperature must be a finite non-negative number"


def test_bodies_that_are_not_a_json_object(parse):
    for body in ['', '[]', '{"temperature":1', '{"temperature":}', '{"a":1,}', '{"a":"unterminated}', '{"a":1} x',
                 '{"a":tru}', '{"a":01}', '{a:1}', '{"a":"bad \\q escape"}', '[' * 100 + ']' * 100]:
        assert parse(body)[0] == FG_ERR_FORMAT, body
    assert parse('{"deep":' + '[' * 60 + ']' * 60 + '}')[0] == FG_OK
