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
