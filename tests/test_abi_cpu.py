"""Host-side checks that need no GPU: the shared library loads and exports every symbol the header declares,
calls fail loudly without a device, and the host-only entry points (rope table, sizes, root files) work."""
import ctypes as C
import os
import re

import numpy as np
import pytest
import torch

from mechta_b200 import _lib, kv

NO_GPU = not torch.cuda.is_available()


def _declared():
    text = open(_lib.HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mkv_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = _lib.lib()
    names = _declared()
    assert len(names) >= 30
    for n in names:
        assert hasattr(L, n), f"{n} is declared in include/mechta_kv.h but not exported"
    assert set(names) == set(_lib.exported_symbols()), "binding table and header disagree"
    assert b"sm_100a" in L.mkv_version()


def _c_prototypes():
    """name -> number of parameters, from the header."""
    text = re.sub(r"/\*.*?\*/", "", open(_lib.HEADER).read(), flags=re.S)
    out = {}
    for m in re.finditer(r"\b(mkv_[a-z0-9_]+)\s*\(([^;{}]*?)\)\s*;", text):
        args = " ".join(m.group(2).split())
        out[m.group(1)] = 0 if args in ("", "void") else len(args.split(","))
    return out


def test_rust_sys_crate_declares_the_whole_abi():
    """rust/mechta-kv-sys/src/lib.rs (the `-sys` crate a Rust host links; it could not be compiled where it was written)
    against include/mechta_kv.h: the same entry points with the same number of arguments, the structs with the same
    fields, and the file is what its generator writes from the header today."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    rs = open(os.path.join(root, "rust", "mechta-kv-sys", "src", "lib.rs")).read()
    rust = {}
    for m in re.finditer(r"pub fn (mkv_[a-z0-9_]+)\(([^)]*)\)", rs):
        args = m.group(2).strip()
        rust[m.group(1)] = 0 if not args else len(args.split(","))
    c = _c_prototypes()
    assert len(c) >= 45
    assert set(rust) == set(c), f"missing in Rust: {sorted(set(c) - set(rust))}; unknown in Rust: {sorted(set(rust) - set(c))}"
    for name, n in c.items():
        assert rust[name] == n, f"{name}: {n} parameters in the header, {rust[name]} in the Rust declaration"
    for sname, fields in (("mkv_verify_item", ["cache", "layer", "first_pos", "pos", "ntok", "q_dev", "out_dev"]),
                          ("mkv_step_in", ["qf_dev", "kb_dev", "vb_dev", "q_norm_dev", "k_norm_dev", "rope_tab_dev", "eps"])):
        body = re.search(r"#\[repr\(C\)\]\s*#\[derive\(Clone, Copy\)\]\s*pub struct %s \{(.*?)\}" % sname, rs, flags=re.S).group(1)
        assert re.findall(r"pub (\w+):", body) == fields
    # the ctypes table agrees on the parameter counts as well
    for name, (_, argtypes) in _lib._SIGS.items():
        assert len(argtypes) == c[name], name
    gen = os.path.join(root, "rust", "mechta-kv-sys", "gen_bindings.py")
    assert subprocess.run([sys.executable, gen, "--check"]).returncode == 0
    # the safe wrapper only calls what the -sys crate declares
    wrapper = open(os.path.join(root, "rust", "mechta-kv", "src", "lib.rs")).read()
    used = set(re.findall(r"sys::(mkv_[a-z0-9_]+)\(", wrapper))
    assert used and used <= set(rust)


@pytest.mark.skipif(not NO_GPU, reason="checks the behaviour without a device")
def test_no_device_is_an_error_not_a_fallback():
    h = C.c_void_p()
    st = _lib.lib().mkv_ctx_create(0, None, C.byref(h))
    assert st == _lib.ERR_CUDA and not h.value
    assert b"no CPU path" in _lib.lib().mkv_last_error()
    with pytest.raises(_lib.MkvError):
        kv.KvContext(0)


def test_rope_table_matches_oracle(oracle):
    for pos in (0, 1, 4096, 65535, 262143):
        assert np.array_equal(kv.rope_table(pos, 4), oracle.rope_tables(pos, 4))


def test_sizes(oracle):
    assert kv.KvFormat.F32.buffer_bytes_for(65536) * 22 == 2_952_790_016  # memcheck.rs:111
    for ctx in (4096, 65536, 131072, 262144):
        for fmt in (0, 1):
            assert kv.need_bytes(ctx, kv.KvFormat(fmt), 11) == oracle.lib().mko_need_bytes_kv(ctx, fmt, 11)
    assert kv.check_ctx(65536) == 65536
    for bad in (0, 4095, 5000, 262144 + 1024):
        with pytest.raises(ValueError):
            kv.check_ctx(bad)


def test_root_key_matches_oracle(oracle):
    toks = np.arange(5000, dtype=np.uint32) * 31 + 7
    assert kv.root_key(toks) == f"{oracle.root_key(toks):016x}"


@pytest.mark.parametrize("fmt", [kv.KvFormat.F16, kv.KvFormat.F32])
def test_root_file_roundtrip_and_reference_layout(tmp_path, fmt):
    n_layers, p = 3, 40
    words = fmt.data_words(p * 512)
    rng = np.random.default_rng(5)
    payload = torch.from_numpy(rng.integers(0, 256, size=2 * n_layers * words * 4, dtype=np.uint8))
    toks = rng.integers(0, 150000, size=p, dtype=np.uint32)
    path = str(tmp_path / "root-test.bin")
    kv.write_root_file(path, toks, kv.Root(p, fmt, n_layers, payload))
    raw = open(path, "rb").read()
    # session.rs:98-106: header, p, n_ssm, n_kv, tokens, then length-prefixed vectors
    assert raw.startswith(b"MECHTA-ROOT-1\n")
    o = 14
    assert np.frombuffer(raw, "<u8", 3, o).tolist() == [p, 0, n_layers]
    o += 24
    assert np.array_equal(np.frombuffer(raw, "<u4", p, o), toks)
    o += 4 * p
    for i in range(2 * n_layers):
        assert int(np.frombuffer(raw, "<u8", 1, o)[0]) == words
        o += 8
        assert raw[o:o + 4 * words] == payload.numpy()[i * 4 * words:(i + 1) * 4 * words].tobytes()
        o += 4 * words
    assert o == len(raw) and not os.path.exists(path + ".tmp")
    t2, r2 = kv.read_root_file(path, fmt, n_layers, pin=False)
    assert np.array_equal(t2, toks) and r2.p == p and torch.equal(r2.payload, payload)


def test_root_file_with_deltanet_states_is_read_and_bad_files_rejected(tmp_path):
    """A file as the reference writes it (n_ssm > 0): states skipped, KV read. Then corrupt variants."""
    fmt, n_layers, p = kv.KvFormat.F16, 2, 8
    words = fmt.data_words(p * 512)
    rng = np.random.default_rng(6)
    toks = rng.integers(0, 1000, size=p, dtype=np.uint32)
    kvw = rng.integers(0, 2**32, size=(2 * n_layers, words), dtype=np.uint64).astype("<u4")
    blob = b"MECHTA-ROOT-1\n" + np.array([p, 2, n_layers], "<u8").tobytes() + toks.tobytes()
    for n in (5, 7, 3, 4):  # 2 ssm + 2 conv vectors
        blob += np.array([n], "<u8").tobytes() + np.zeros(n, "<f4").tobytes()
    for i in range(2 * n_layers):
        blob += np.array([words], "<u8").tobytes() + kvw[i].tobytes()
    path = str(tmp_path / "ref.bin")
    open(path, "wb").write(blob)
    t2, r2 = kv.read_root_file(path, fmt, n_layers, pin=False)
    assert np.array_equal(t2, toks) and r2.payload.numpy().tobytes() == kvw.tobytes()
    for bad in (b"MECHTA-ROOT-2\n" + blob[14:], blob[:-10], blob[:30]):
        open(path, "wb").write(bad)
        with pytest.raises(_lib.MkvError) as e:
            kv.read_root_file(path, fmt, n_layers, pin=False)
        assert e.value.status == _lib.ERR_FORMAT
    open(path, "wb").write(blob)
    with pytest.raises(_lib.MkvError) as e:
        kv.read_root_file(path, fmt, n_layers + 1, pin=False)
    assert e.value.status == _lib.ERR_FORMAT
    with pytest.raises(_lib.MkvError) as e:
        kv.read_root_file(str(tmp_path / "missing.bin"), fmt, n_layers, pin=False)
    assert e.value.status == _lib.ERR_IO
