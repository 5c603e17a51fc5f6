"""CPU checks of the reference-kernel shim (oracle/_ref/libref_cuda.so, built from the reference's own
src/backend/cuda/kernels.cu): the library loads, exports its launchers, and restates the reference's tile-shape
rule (src/backend/cuda.zig:1940-1987) on the cases that file's comments name. No kernel runs here."""
import pytest

from oracle import ref_cuda

pytestmark = pytest.mark.skipif(not ref_cuda.available(), reason="oracle/_ref/libref_cuda.so was not built")


def test_library_exports_launchers():
    L = ref_cuda.lib()
    for name in ("refk_gemv", "refk_mul_mm", "refk_plan"):
        assert hasattr(L, name)


def test_launch_plan_known_cases():
    q6, q4 = ref_cuda.FORMATS["q6_k"], ref_cuda.FORMATS["q4_k"]
    # 64 N64 blocks on 76 SMs are below the 7/8 cutoff (67) and split K in two (cuda.zig:1956-1957)
    assert ref_cuda.plan(q4, 76, 1, 4096, 1024) == (64, 2)
    # 24 blocks on 76 SMs: Q6_K splits three ways, Q4_K two (cuda.zig:1960-1966)
    assert ref_cuda.plan(q6, 76, 1, 1536, 1024) == (64, 3)
    assert ref_cuda.plan(q4, 76, 1, 1536, 1024) == (64, 2)
    # the split never exceeds k / 128
    assert ref_cuda.plan(q4, 76, 1, 1536, 128) == (32, 1)
    # a full grid keeps N64 tiles and one K range; the grouped entry never splits (cuda.zig:2303)
    assert ref_cuda.plan(q4, 148, 16, 14336, 4096) == (64, 1)
    assert ref_cuda.plan(q4, 148, 1, 1536, 1024, allow_split_k=False) == (32, 1)
    # launches that refuse before any CUDA call: m outside 1..8 on the decode kernel
    assert ref_cuda.lib().refk_gemv(q4, None, None, None, 256, 4, 9, 144, None) == 1


def test_tile_tables_follow_the_reference_layout():
    # {expert, group base, group rows, tile index}: src/llm/gemma/moe.zig:773-787, src/backend/cuda.zig:3170-3183
    assert ref_cuda.grouped_tiles([1, 7, 33, 40]) == [[0, 0, 1, 0], [1, 1, 7, 0], [2, 8, 33, 0], [2, 8, 33, 1], [3, 41, 40, 0], [3, 41, 40, 1]]
    assert ref_cuda.grouped_tiles([0, 5]) == [[1, 0, 5, 0]]
    assert ref_cuda.dense_tiles(65) == [[0, 0, 65, 0], [0, 0, 65, 1], [0, 0, 65, 2]]
