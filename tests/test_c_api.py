"""The C API and its C++ owners, driven from compiled C / C++ programs that host the runtime themselves (reference:
test/c_api_tests.cpp).  The programs print `key: value` lines; the values are compared with what the Python API gives for
the same model and options."""
import os
import shutil
import subprocess
import sys
import sysconfig

import numpy as np
import pytest

import onnxruntime_genai_b200 as og
from helpers import tiny_model_dir
from onnxruntime_genai_b200.build_native import C_API_DIR, build_c_api

HERE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "c_api")

pytestmark = pytest.mark.skipif(shutil.which("gcc") is None, reason="no C compiler")


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    d, _ = tiny_model_dir(str(tmp_path_factory.mktemp("capi_model")), std=0.3)
    return d


def _compile(tmp_path, source, cxx):
    build_c_api()
    exe = str(tmp_path / os.path.splitext(source)[0])
    cc = ["g++", "-std=c++17"] if cxx else ["gcc", "-std=c11"]
    subprocess.run([*cc, "-Wall", "-O1", "-I" + C_API_DIR, os.path.join(HERE, source), "-o", exe, "-L" + C_API_DIR, "-logb200_genai",
                    "-Wl,-rpath," + C_API_DIR], check=True, capture_output=True, text=True)
    return exe


def _run(exe, model_dir):
    env = dict(os.environ, OGB_PYTHON=sys.executable)
    r = subprocess.run([exe, model_dir], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout + r.stderr
    out = {}
    for line in r.stdout.splitlines():
        k, _, v = line.partition(":")
        out[k.strip()] = v.strip()
    return out, r.stderr


def _greedy(model_dir, max_length, prompt="hello world"):
    model = og.Model(model_dir)
    tok = og.Tokenizer(model)
    params = og.GeneratorParams(model)
    params.set_search_options(max_length=max_length, do_sample=False)
    gen = og.Generator(model, params)
    gen.append_tokens(tok.encode(prompt))
    while not gen.is_done():
        gen.generate_next_token()
    return " ".join(str(int(t)) for t in gen.get_sequence(0)), len(tok.encode(prompt))


def test_c_program_generates_streams_batches_and_shuts_down(tmp_path, model_dir):
    out, err = _run(_compile(tmp_path, "c_api_test.c", cxx=False), model_dir)
    want, n_prompt = _greedy(model_dir, 24)
    assert out["bad_model_error"] == "yes" and out["bad_option_error"] == "yes"
    assert out["model_type"] == "llama" and out["max_length"] == "24"
    assert out["greedy"] == want and out["after_rewind"] == want
    assert out["token_count"] == "24" and out["generated"] == str(24 - n_prompt)
    assert out["streamed_prompt"] == "hello world" and out["decoded_prompt"] == "hello world"
    assert out["logits"] == "rank 3 rows 1 type 1"
    assert out["named_tensors"] == "1 value 6"
    # the engine emits the continuation only (same greedy tokens as the generator)
    assert out["engine_0"] == " ".join(want.split()[n_prompt:])
    assert out["engine_1"] == " ".join(_greedy(model_dir, 24, "The quick brown fox")[0].split()[len(og.Tokenizer(og.Model(model_dir)).encode("The quick brown fox")):])
    assert out["engine_complete_0"] == "yes" and out["engine_complete_1"] == "yes"
    # every handle was destroyed before the first shutdown; the library works again afterwards; a leaked handle is reported
    assert out["live_before_shutdown"] == "0"
    assert out["after_shutdown"] == _greedy(model_dir, 16)[0]
    assert out["live_with_leak"] == "1"
    assert "OgaSequences: 1" in err and err.count("Still alive") == 1


def test_cpp_owners(tmp_path, model_dir):
    out, err = _run(_compile(tmp_path, "cpp_api_test.cpp", cxx=True), model_dir)
    want, n_prompt = _greedy(model_dir, 24)
    assert out["bad_model_error"] == "yes"
    assert out["greedy"] == want and out["logits_rank"] == "3"
    assert out["engine_0"] == " ".join(want.split()[n_prompt:]) and out["engine_rows_equal"] == "yes"
    assert "Still alive" not in err


def test_library_joins_a_running_interpreter(model_dir):
    """Loaded with ctypes into this process, the library uses the interpreter that is already there."""
    import ctypes
    lib = ctypes.CDLL(build_c_api())
    P = ctypes.c_void_p
    lib.OgaResultGetError.restype = ctypes.c_char_p
    lib.OgaResultGetError.argtypes = [P]
    lib.OgaCreateModel.restype = P
    lib.OgaCreateModel.argtypes = [ctypes.c_char_p, ctypes.POINTER(P)]
    lib.OgaModelGetType.restype = P
    lib.OgaModelGetType.argtypes = [P, ctypes.POINTER(ctypes.c_char_p)]
    lib.OgaDestroyModel.argtypes = [P]
    lib.OgaLiveHandleCount.restype = ctypes.c_size_t
    m = P()
    r = lib.OgaCreateModel(model_dir.encode(), ctypes.byref(m))
    assert not r, lib.OgaResultGetError(r)
    s = ctypes.c_char_p()
    assert not lib.OgaModelGetType(m, ctypes.byref(s))
    assert s.value == b"llama"
    assert lib.OgaLiveHandleCount() == 1
    lib.OgaDestroyModel(m)
    assert lib.OgaLiveHandleCount() == 0


def test_streaming_processor_through_the_c_api(tmp_path):
    """OgaCreateStreamingProcessor / Process / Flush / SetOption / GetOption over a speech-transducer model: the frames that come
    back through the C entry points equal the Python front end's, a chunk that completes no frame returns a null tensor set."""
    import ctypes
    import numpy as np
    import torch
    import onnxruntime_genai_b200 as og
    from onnxruntime_genai_b200 import streaming
    from onnxruntime_genai_b200.models.encoder import EncoderConfig
    from onnxruntime_genai_b200.models.transducer import TransducerConfig, export_transducer
    enc = EncoderConfig(kind="audio", hidden_size=32, num_layers=1, num_heads=4, intermediate_size=64, num_mel_bins=16, max_source_positions=200)
    cfg = TransducerConfig(vocab_size=11, blank_id=10, encoder_hidden=32, pred_hidden=16, pred_layers=1, joint_hidden=16, tdt_durations="0,1,2")
    g = torch.Generator().manual_seed(0)
    vsd = {n: torch.randn(s, generator=g) * 0.3 for n, s in streaming.vad_weight_shapes(16000, 8).items()}
    d = str(tmp_path)
    streaming.export_vad(d, vsd)
    export_transducer(cfg, enc, d, "parakeet_tdt", "fp32", "cpu", num_mels=16, chunk_samples=1600,
                      vad={"filename": "vad.onnx", "threshold": 0.0, "silence_duration_ms": 300, "prefix_padding_ms": 100})
    lib = ctypes.CDLL(build_c_api())
    P = ctypes.c_void_p
    lib.OgaResultGetError.restype = ctypes.c_char_p
    lib.OgaResultGetError.argtypes = [P]
    for name, args in (("OgaCreateModel", [ctypes.c_char_p, ctypes.POINTER(P)]), ("OgaCreateStreamingProcessor", [P, ctypes.POINTER(P)]),
                       ("OgaStreamingProcessorProcess", [P, ctypes.POINTER(ctypes.c_float), ctypes.c_size_t, ctypes.POINTER(P)]),
                       ("OgaStreamingProcessorFlush", [P, ctypes.POINTER(P)]),
                       ("OgaStreamingProcessorSetOption", [P, ctypes.c_char_p, ctypes.c_char_p]),
                       ("OgaStreamingProcessorGetOption", [P, ctypes.c_char_p, ctypes.POINTER(ctypes.c_char_p)]),
                       ("OgaNamedTensorsGet", [P, ctypes.c_char_p, ctypes.POINTER(P)]), ("OgaTensorGetShapeRank", [P, ctypes.POINTER(ctypes.c_size_t)]),
                       ("OgaTensorGetShape", [P, ctypes.POINTER(ctypes.c_int64), ctypes.c_size_t]), ("OgaTensorGetData", [P, ctypes.POINTER(P)])):
        getattr(lib, name).restype = P
        getattr(lib, name).argtypes = args
    for name in ("OgaDestroyModel", "OgaDestroyStreamingProcessor", "OgaDestroyNamedTensors", "OgaDestroyTensor", "OgaDestroyResult"):
        getattr(lib, name).argtypes = [P]
    ok = lambda r: (not r) or pytest.fail(lib.OgaResultGetError(r).decode())
    m, sp = P(), P()
    ok(lib.OgaCreateModel(d.encode(), ctypes.byref(m)))
    ok(lib.OgaCreateStreamingProcessor(m, ctypes.byref(sp)))
    val = ctypes.c_char_p()
    ok(lib.OgaStreamingProcessorGetOption(sp, b"silence_duration_ms", ctypes.byref(val)))
    assert float(val.value) == 300.0
    ok(lib.OgaStreamingProcessorSetOption(sp, b"threshold", b"0.0"))
    r = lib.OgaStreamingProcessorSetOption(sp, b"no_such_option", b"1")
    assert r and b"unknown streaming option" in lib.OgaResultGetError(r)
    lib.OgaDestroyResult(r)

    audio = (np.random.RandomState(0).randn(1600 * 3 + 700) * 0.1).astype(np.float32)
    ref = og.Model(d).create_streaming_processor()
    ref.set_option("threshold", "0.0")

    def frames_of(nt):
        t = P()
        ok(lib.OgaNamedTensorsGet(nt, b"audio_features", ctypes.byref(t)))
        rank = ctypes.c_size_t()
        ok(lib.OgaTensorGetShapeRank(t, ctypes.byref(rank)))
        shape = (ctypes.c_int64 * rank.value)()
        ok(lib.OgaTensorGetShape(t, shape, rank.value))
        data = P()
        ok(lib.OgaTensorGetData(t, ctypes.byref(data)))
        n = int(np.prod(list(shape)))
        arr = np.ctypeslib.as_array(ctypes.cast(data, ctypes.POINTER(ctypes.c_float)), shape=(n,)).reshape(list(shape)).copy()
        lib.OgaDestroyTensor(t)
        return arr

    for s0, n in ((0, 300), (300, 1600 * 3 - 300), (1600 * 3, 700)):
        piece = audio[s0:s0 + n]
        nt = P()
        ok(lib.OgaStreamingProcessorProcess(sp, piece.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), len(piece), ctypes.byref(nt)))
        want = ref.process(piece)
        if want is None:
            assert not nt
        else:
            got = frames_of(nt)
            assert got.shape == (1,) + want.shape
            np.testing.assert_allclose(got[0], want, rtol=1e-6, atol=1e-6)
            lib.OgaDestroyNamedTensors(nt)
    nt = P()
    ok(lib.OgaStreamingProcessorFlush(sp, ctypes.byref(nt)))
    want = ref.flush()
    assert (want is None) == (not nt)
    if nt:
        np.testing.assert_allclose(frames_of(nt)[0], want, rtol=1e-6, atol=1e-6)
        lib.OgaDestroyNamedTensors(nt)
    lib.OgaDestroyStreamingProcessor(sp)
    lib.OgaDestroyModel(m)
