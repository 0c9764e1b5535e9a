"""CPU-side checks of the C-ABI library: it loads, exports every symbol the
header declares, and its host-only entry points behave.  No kernel is launched."""
import ctypes as C
import os
import re

import pytest

from conftest import ROOT


def declared_functions():
    text = open(os.path.join(ROOT, "include", "moe_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(moe_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg.lib()
    names = declared_functions()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/moe_b200.h but not exported"
    assert set(pkg.EXPORTS) <= set(names)


def test_shard_ranges_cover_and_follow_the_reference_split(pkg):
    for D, tp in [(2880, 1), (2880, 2), (2880, 4), (2880, 8), (96, 3), (64, 2), (320, 4), (160, 3)]:
        pos = 0
        lens = []
        for r in range(tp):
            s, n = pkg.shard_range(D, tp, r)
            assert s == pos and n > 0 and n % 8 == 0
            pos += n
            lens.append(n)
        assert pos == D
        assert max(lens) - min(lens) <= 32
    # even split as mlp2_shard_input of the reference whenever it yields whole gate/up row groups
    assert [pkg.shard_range(2880, 4, r) for r in range(4)] == [(0, 720), (720, 720), (1440, 720), (2160, 720)]
    assert [pkg.shard_range(2880, 8, r)[1] for r in range(8)] == [360] * 8
    # otherwise whole 32-element scale blocks are dealt out
    assert [pkg.shard_range(160, 3, r) for r in range(3)] == [(0, 64), (64, 64), (128, 32)]
    with pytest.raises(pkg.MoeError):
        pkg.shard_range(2880, 4, 4)
    with pytest.raises(pkg.MoeError):
        pkg.shard_range(100, 2, 0)   # not a multiple of 32


def test_create_rejects_bad_config_and_fails_loudly_without_gpu(pkg):
    lib = pkg.lib()
    h = C.c_void_p()
    bad = pkg.MoeConfig(2880, 2880, 128, 4, 1, 7.0, 1.702, 0, 1, 0, 0, 0)      # max_rows = 0
    assert lib.moe_create(C.byref(bad), C.byref(h)) == 1 and not h
    bad = pkg.MoeConfig(2880, 2890, 128, 4, 1, 7.0, 1.702, 64, 1, 0, 0, 0)     # D % 32 != 0
    assert lib.moe_create(C.byref(bad), C.byref(h)) == 1 and not h
    bad = pkg.MoeConfig(2880, 2880, 128, 4, 1, 7.0, 1.702, 64, 2, 2, 0, 0)     # rank outside group
    assert lib.moe_create(C.byref(bad), C.byref(h)) == 1 and not h
    import torch
    if not torch.cuda.is_available():
        # no CPU path exists: creation must fail with a CUDA error, not fall back
        with pytest.raises(pkg.MoeError) as ei:
            pkg.MoeBlock(64, 64, 8, max_rows=8)
        assert ei.value.code in (2, 7)


def test_error_strings(pkg):
    lib = pkg.lib()
    assert lib.moe_strerror(0) == b"ok"
    assert b"wait" in lib.moe_strerror(4)
    assert lib.moe_last_error(None) == b"null handle"


def test_algorithmic_work_matches_published_formula(synth):
    # 199 065 600 flop per token + router; bytes = experts * 13 236 480 + rows in/out + router weights
    flops, nbytes = synth.algorithmic_work(1856, 2880, 2880, 128, 4, 128)
    assert flops == 1856 * (199065600 + 2 * 2880 * 128)
    assert synth.weight_bytes_per_expert(2880, 2880) == 13236480
    assert nbytes == 128 * 13236480 + 1856 * 2880 * 4 + 128 * 2880 * 4


def test_cpp_shim_compiles_and_links(tmp_path):
    """include/moe_b200_shim.hpp (the reference's entry-point names on top of the C ABI) builds
    with the host compiler and its host-only helpers agree with the library."""
    import shutil
    import subprocess
    src = tmp_path / "shim.cpp"
    src.write_text(r"""
#include <thread>
#include "moe_b200_shim.hpp"
// every name of the reference's MoE boundary must exist with the reference's parameter lists
static void (*p_moe_gpu)(GPUTransformer *, int, int, int, cudaStream_t) = &moe_gpu;
static void (*p_moe_gpu_120b)(GPUTransformer *, int, int, int, cudaStream_t) = &moe_gpu_120b;
static void (*p_allgather)(void *, const void *, int, int, void *const[], const TPGroup &, cudaStream_t) = &ring_allgather_rows_bf16;
static void (*p_allreduce)(void *, void *const[], size_t, void *, const TPGroup &, cudaStream_t) = &ring_allreduce_sum_bf16;
int main() {
  TPGroup tp; tp_init(tp, 8, 5, 4); int s, n; mlp1_shard(5760, 4, 1, s, n);
  int a, b; mlp2_shard_input(2880, 4, 3, a, b);
  GPUTransformer gt = {}; gt.config.hidden_dim = 2880; gt.state.x = nullptr; gt.weights.rms_ffn_w = nullptr;
  // tp_group_barrier: four host threads of one group meet three times
  TPGroup g[4]; int order = 0;
  for (int r = 0; r < 4; ++r) tp_init(g[r], 4, r, 4);
  std::thread th[4];
  for (int r = 0; r < 4; ++r) th[r] = std::thread([&, r] { for (int i = 0; i < 3; ++i) { tp_group_barrier(g[r]); __sync_fetch_and_add(&order, 1); tp_group_barrier(g[r]); } });
  for (auto &t : th) t.join();
  return (tp.group_id == 1 && tp.rank_in_group == 1 && tp.group_devs[3] == 7 && s == 1440 && n == 1440
          && a == 2160 && b == 720 && order == 12 && p_moe_gpu && p_moe_gpu_120b && p_allgather && p_allreduce) ? 0 : 1; }
""")
    gxx = shutil.which("g++")
    if gxx is None or not os.path.exists("/usr/local/cuda/include/cuda_runtime.h"):
        pytest.skip("no host compiler or CUDA headers")
    exe = tmp_path / "shim"
    libdir = os.path.join(ROOT, "gpt-oss_b200")
    subprocess.run([gxx, "-std=c++17", "-pthread", "-I" + os.path.join(ROOT, "include"), "-I/usr/local/cuda/include", str(src),
                    "-L" + libdir, "-lmoe_b200", "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath," + libdir,
                    "-Wl,-rpath,/usr/local/cuda/lib64", "-o", str(exe)], check=True)
    assert subprocess.run([str(exe)]).returncode == 0
