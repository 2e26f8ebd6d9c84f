"""The C++ operator surface (include/*.hpp: OperatorRegistry, OperatorFactory, UnifiedOp,
FlashAttnOperator, KVCachePool) compiled with g++ against libinfer_b200.so, no torch types.
Host-only checks run everywhere; the GPU run exchanges raw files with a small C++ driver and is
checked against the CPU oracle."""
import shutil
import struct
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

from gpu_util import ATOL_BF16, RTOL_BF16, assert_close
from infer_b200 import _lib
from oracle import paged_kv_oracle as oracle

ROOT = Path(__file__).resolve().parent.parent
CUDA = Path("/usr/local/cuda")


@pytest.fixture(scope="module")
def surface_binary(tmp_path_factory):
    if shutil.which("g++") is None or not (CUDA / "include" / "cuda_runtime.h").exists():
        pytest.skip("g++ or the CUDA headers are not available")
    out = tmp_path_factory.mktemp("cpp") / "surface_test"
    lib_dir = _lib.LIB_PATH.parent
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", f"-I{ROOT / 'include'}", f"-I{CUDA / 'include'}",
           str(ROOT / "tests" / "cpp" / "surface_test.cpp"), "-o", str(out), f"-L{lib_dir}", "-linfer_b200",
           f"-L{CUDA / 'lib64'}", "-lcudart", "-lpthread", f"-Wl,-rpath,{lib_dir}", f"-Wl,-rpath,{CUDA / 'lib64'}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return out


def test_cpp_surface_host_logic(surface_binary):
    res = subprocess.run([str(surface_binary), "cpu"], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "surface cpu ok" in res.stdout


@pytest.mark.gpu
def test_cpp_surface_on_gpu(surface_binary, tmp_path):
    gen = torch.Generator().manual_seed(77)
    b, hq, hkv, nb, s = 5, 16, 8, 24, 200
    lens = [1, 300, 513, 256, 777]
    q = torch.randn(b, hq, 128, generator=gen).bfloat16()
    ks = [torch.randn(n, hkv, 128, generator=gen).bfloat16() for n in lens]
    vs = [torch.randn(n, hkv, 128, generator=gen).bfloat16() for n in lens]
    Q = torch.randn(1, hq, s, 128, generator=gen).bfloat16()
    K = torch.randn(1, hkv, s, 128, generator=gen).bfloat16()
    V = torch.randn(1, hkv, s, 128, generator=gen).bfloat16()
    raw = lambda t: t.contiguous().view(torch.int16).numpy().tobytes()
    blob = struct.pack(f"{5 + b}i", b, hq, hkv, nb, s, *lens) + raw(q)
    for k, v in zip(ks, vs):
        blob += raw(k) + raw(v)
    blob += raw(Q) + raw(K) + raw(V)
    fin, fout = tmp_path / "in.bin", tmp_path / "out.bin"
    fin.write_bytes(blob)
    res = subprocess.run([str(surface_binary), "gpu", str(fin), str(fout)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    out = fout.read_bytes()
    w = struct.unpack("i", out[:4])[0]
    bt = torch.tensor(np.frombuffer(out[4:4 + 4 * b * w], dtype=np.int32).reshape(b, w).copy())
    at = 4 + 4 * b * w
    got = torch.from_numpy(np.frombuffer(out[at:at + b * hq * 256], dtype=np.int16).copy()).view(torch.bfloat16).view(b, hq, 128)
    at += b * hq * 256
    dense = torch.from_numpy(np.frombuffer(out[at:at + hq * s * 256], dtype=np.int16).copy()).view(torch.bfloat16).view(1, hq, s, 128)
    # pages: first halves of every sequence in order, then second halves (FIFO free list)
    assert w == 4 and bt[4].tolist()[:4] != [-1] * 4
    used = [p for row in bt.tolist() for p in row if p >= 0]
    assert sorted(used) == list(range(len(used)))                    # every page handed out once, lowest ids first
    # rebuild the pools on the CPU with the block tables the C++ pool produced
    kc = torch.zeros(nb, 256, hkv, 128, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    for i, n in enumerate(lens):
        slots = torch.tensor([int(bt[i, p // 256]) * 256 + p % 256 for p in range(n)], dtype=torch.int32)
        oracle.store_kvcache(ks[i], vs[i], kc, vc, slots)
    want = oracle.paged_decode(q, kc, vc, torch.tensor(lens, dtype=torch.int32), bt, 128 ** -0.5)
    assert_close(got, want, ATOL_BF16, RTOL_BF16, "C++ surface: append + paged decode")
    assert_close(dense, oracle.dense_causal(Q, K, V), ATOL_BF16, RTOL_BF16, "C++ surface: UnifiedOp::attention")


@pytest.fixture(scope="module")
def block_manager_binary(tmp_path_factory):
    if shutil.which("g++") is None:
        pytest.skip("g++ is not available")
    out = tmp_path_factory.mktemp("cppbm") / "block_manager_test"
    res = subprocess.run(["g++", "-std=c++17", "-O2", "-Wall", f"-I{ROOT / 'include'}",
                          str(ROOT / "tests" / "cpp" / "block_manager_test.cpp"), "-o", str(out)], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return out


def test_native_xxh64_matches_xxhash(block_manager_binary):
    """The header's XXH64 against the xxhash package the reference uses, on the exact byte
    strings its BlockManager hashes (int64 token ids, optional 8-byte prefix) and odd lengths."""
    import xxhash
    rng = np.random.default_rng(3)
    cases, want = [], []
    for n in (0, 1, 3, 4, 5, 31, 256, 257):
        toks = rng.integers(0, 2 ** 40, size=n).tolist()
        for prefix in (None, int(rng.integers(0, 2 ** 63)) * 2 + 1):
            h = xxhash.xxh64()
            if prefix is not None:
                h.update(prefix.to_bytes(8, "little"))
            h.update(np.array(toks, dtype=np.int64).tobytes())
            want.append(h.intdigest())
            cases.append(" ".join(map(str, [n] + toks + ([prefix] if prefix is not None else []))))
    res = subprocess.run([str(block_manager_binary), "hash"], input="\n".join(cases) + "\n", capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    assert [int(x) for x in res.stdout.split()] == want


def test_native_block_manager_matches_reference(block_manager_binary, golden, tmp_path):
    """The same scripted engine life as tests/golden (prefill with shared prefixes, decode growth
    across page boundaries, frees, digest revival) through the C++ allocator: page lists, cache
    hits, reference counts and free-list order equal the reference's at every snapshot."""
    import json
    g = golden["allocator"]
    lines = [f"N {g['num_blocks']} {g['block_size']}"]
    for p in g["prompts"]:
        lines.append("A " + " ".join(map(str, [len(p)] + p)))
    lines.append("S")
    for toks in g["new_tokens"]:
        for i, t in enumerate(toks):
            lines.append(f"T {i} {t}")
        lines.append("S")
    lines += ["D 0", "D 2", "S"]
    late = g["late_prompt"]
    lines += ["A " + " ".join(map(str, [len(late)] + late)), "S"]
    scen = tmp_path / "scenario.txt"
    scen.write_text("\n".join(lines) + "\n")
    res = subprocess.run([str(block_manager_binary), str(scen)], capture_output=True, text=True, timeout=60)
    assert res.returncode == 0, res.stderr
    snaps = [json.loads(l) for l in res.stdout.splitlines()]
    assert len(snaps) == len(g["events"])
    for got, want in zip(snaps, g["events"]):
        for key in ("tables", "cached", "lens", "ref_counts", "free"):
            assert got[key] == want[key], (want["tag"], key)
