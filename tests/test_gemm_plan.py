"""How the tensor-core matrix product is cut into tiles, splits and waves: decisions of the host code in
csrc/gemm_tc.cu, asked through `ops.gemm_tc_describe` for a device of 148 SMs.  Nothing is launched, so this runs
without a GPU; it needs nvcc to build the library and is skipped without it."""
import pytest

from hymt2sharp_b200.kernels import build

STORE, ADD, SWIGLU, QKV = 0, 1, 2, 3
SMS = 148


@pytest.fixture(scope="module")
def describe():
    try:
        build.find_nvcc()
    except Exception as err:   # no compiler here: the library cannot be built
        pytest.skip(f"nvcc is not available: {err}")
    from hymt2sharp_b200.kernels import ops
    return lambda T, N, K, epi: ops.gemm_tc_describe(T, N, K, epi, sm_count=SMS)


def test_few_tokens_put_the_weight_rows_on_the_128_row_side(describe):
    for tokens, width in ((1, 16), (16, 16), (17, 32), (33, 64), (64, 64), (65, 128), (128, 128)):
        plan = describe(tokens, 6144, 2048, SWIGLU)
        assert plan["swapped"] and not plan["persistent"] and plan["tile_width"] == width
    assert not describe(129, 6144, 2048, SWIGLU)["swapped"]


@pytest.mark.parametrize("N, K, epi", [(6144, 2048, SWIGLU), (2048, 6144, ADD), (2048, 2048, ADD), (3072, 2048, QKV),
                                       (120818, 2048, STORE), (392, 264, STORE), (8192, 3072, SWIGLU), (4096, 14336, ADD)])
def test_the_cut_of_k_never_depends_on_the_number_of_tokens(describe, N, K, epi):
    """Or a sequence's logits would depend on what else is in the batch.  This holds inside the orientation for few
    tokens (up to 128).  From 129 tokens on the orientation flips and K is not cut at all: partial sums folded in
    split order become one unsplit accumulation, so in bfloat16 a token's result may differ in the last bit between
    a 128-token and a 129-token step.  Bit-for-bit independence of the batch is a property of the 32-bit path (the
    CUDA-core product sums in ascending K whatever the number of tokens is); the bfloat16 path promises it within
    rounding."""
    assert not describe(129, N, K, epi)["swapped"] and describe(129, N, K, epi)["k_splits"] == 1
    plans = [describe(T, N, K, epi) for T in (1, 2, 8, 16, 17, 40, 64, 100, 128)]
    assert len({p["k_splits"] for p in plans}) == 1
    assert all(p["k_splits"] <= 8 for p in plans)           # a portable cluster
    assert all(p["ctas"] == p["tiles"] * p["k_splits"] for p in plans)


def test_a_product_with_few_tiles_is_cut_to_about_one_wave(describe):
    down = describe(8, 2048, 6144, ADD)      # 16 tiles of 128 features
    assert down["tiles"] == 16 and down["k_splits"] == 8 and down["cluster"]
    gate_up = describe(8, 6144, 2048, SWIGLU)   # 48 tiles, wide stages: the splits fold through memory
    assert gate_up["k_splits"] == 3 and not gate_up["cluster"] and gate_up["ctas"] <= SMS
    head = describe(8, 120818, 2048, STORE)  # 944 tiles: no cut
    assert head["k_splits"] == 1 and head["tiles"] == 944


def test_more_than_128_tokens_always_run_the_persistent_kernel(describe):
    for T in (129, 300, 1536, 2048, 4096, 16384):
        for N, K, epi in ((2048, 2048, ADD), (2048, 6144, ADD), (6144, 2048, SWIGLU), (3072, 2048, STORE), (3072, 2048, QKV)):
            plan = describe(T, N, K, epi)
            assert plan["persistent"] and not plan["swapped"] and plan["k_splits"] == 1
            assert plan["ctas"] == min(plan["tiles"], SMS)


def test_65_to_128_tokens_of_a_split_product_are_two_tiles_of_64_that_fold_as_clusters(describe):
    for N, K, epi in ((2048, 2048, ADD), (2048, 6144, ADD), (3072, 2048, STORE), (3072, 2048, QKV)):
        at64, at100 = describe(64, N, K, epi), describe(100, N, K, epi)
        assert at64["tile_width"] == 64 and at64["cluster"]
        assert at100["tile_width"] == 64 and at100["cluster"] and at100["tiles"] == 2 * at64["tiles"]
        assert at100["k_splits"] == at64["k_splits"]
    assert describe(100, 120818, 2048, STORE)["tile_width"] == 128      # enough tiles: the weights are read once
    assert describe(100, 6144, 2048, SWIGLU)["tile_width"] == 128       # two accumulators: folds through memory anyway


def test_prompt_sized_products_fill_whole_waves(describe):
    # the sizes of the 1.8B model at 2,048 tokens
    gate_up = describe(2048, 6144, 2048, SWIGLU)
    assert gate_up["persistent"] and gate_up["tile_width"] == 224 and gate_up["tiles"] == 880 and gate_up["ctas"] == SMS
    qkv = describe(2048, 3072, 2048, QKV)
    assert qkv["persistent"] and qkv["tile_width"] == 128          # one head a tile up to a few thousand tokens
    assert describe(8192, 3072, 2048, QKV)["tile_width"] == 256    # two heads beyond
    # adding into the residual: one wave of 240-wide tiles at 2,048 tokens (144 of them), every SM busy at 4,096
    for K in (2048, 6144):
        small, large = describe(2048, 2048, K, ADD), describe(4096, 2048, K, ADD)
        assert small["persistent"] and small["tile_width"] == 240 and small["ctas"] == 144
        assert large["persistent"] and large["ctas"] == SMS


@pytest.mark.parametrize("T", [129, 300, 512, 1000, 2048, 5000, 16384])
@pytest.mark.parametrize("N, K, epi", [(6144, 2048, SWIGLU), (3072, 2048, STORE), (3072, 2048, QKV), (896, 256, QKV),
                                       (8192, 3072, SWIGLU), (777, 264, STORE)])
def test_the_width_of_a_persistent_tile_is_one_the_kernel_takes(describe, T, N, K, epi):
    plan = describe(T, N, K, epi)
    assert plan["persistent"] and 128 <= plan["tile_width"] <= 256
    step = {SWIGLU: 32, QKV: 128}.get(epi, 16)   # gate and up halves in chunks of 16 columns; whole heads; chunks of 16
    assert plan["tile_width"] % step == 0
    out_cols = plan["tile_width"] // 2 if epi == SWIGLU else plan["tile_width"]
    assert plan["tiles"] == -(-T // 128) * -(-N // out_cols)
    assert plan["ctas"] == min(plan["tiles"], SMS)
    assert plan["stages"] >= 4                    # the ring: 224 KB of shared memory
    # never more waves than the widest tile would need
    widest = -(-T // 128) * -(-N // (128 if epi == SWIGLU else 256))
    assert -(-plan["tiles"] // SMS) * plan["tile_width"] <= -(-widest // SMS) * 256 * 1.3


def test_the_pieces_of_a_rows_sum_of_squares_do_not_follow_the_tile_width(describe):
    """A product that adds into the residual leaves the rows' sums of squares behind in pieces for the norm after it.  For
    prompts the pieces are per 16 features whatever tile width the step's tokens gave the plan (a piece per tile made the
    last bit of a row's scale depend on what else was in the step); steps of few tokens leave one per tile of 128 weight
    rows, and a product that does not add leaves none."""
    from hymt2sharp_b200.kernels import ops
    widths = set()
    for T in (129, 300, 1470, 2048, 16384):
        widths.add(describe(T, 2048, 6144, ADD)["tile_width"])
        assert ops.gemm_tc_norm_tiles(T, 2048, 6144, ADD) == 2048 // 16
        assert ops.gemm_tc_norm_tiles(T, 2056, 2048, ADD) == 129          # a last piece of 8 features
    assert len(widths) >= 3, widths
    for T in (1, 8, 64, 128):
        assert ops.gemm_tc_norm_tiles(T, 2048, 6144, ADD) == 2048 // 128
    assert ops.gemm_tc_norm_tiles(2048, 6144, 2048, SWIGLU) == 0
