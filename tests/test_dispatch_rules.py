"""The host-side rules that choose how a product is cut: whatever the sizes, the pieces of k they
ask for are ones the kernels accept (no empty piece, whole 64-element blocks), and the rules stay
within the bounds their comments state.  Pure arithmetic: runs without a GPU."""
import itertools

from tokenizer_b200.parts import gemm_bf16 as rules

ROWS = [1, 7, 16, 17, 33, 64, 100, 128, 129, 256, 300, 512, 777, 1024, 1536, 2048, 3000, 4096, 9000]
WIDTHS = [8, 64, 100, 128, 132, 256, 896, 1152, 1536, 4864, 9728, 20000]
DEPTHS = [8, 64, 72, 128, 264, 896, 1032, 2048, 4864, 8192]


def pieces_are_whole(K, pieces):
    """What the tile kernels check: with pieces of ceil(k_blocks / pieces) blocks, none is empty."""
    k_blocks = -(-K // 64)
    per = -(-k_blocks // pieces)
    return pieces >= 1 and (pieces - 1) * per < k_blocks


SIZES = list(itertools.product(ROWS, WIDTHS, DEPTHS))


def test_pieces_of_k_for_tile_products():
    cut = 0
    for M, N, K in SIZES:
        pieces = rules.choose_tile_k_splits(M, N, K)
        assert 1 <= pieces <= 8 and pieces_are_whole(K, pieces), (M, N, K, pieces)
        if pieces > 1:
            cut += 1
            # the consumer adds every plane: at most 8 MB of them, none of more than 4 MB
            assert M * N * 4 <= 4_000_000 and pieces * M * N * 4 <= 8_000_000, (M, N, K, pieces)
            assert N % 4 == 0                                    # planes are stored in 16-byte TMA rows
            assert -(-M // 128) * -(-N // 128) * 2 <= 148        # only when the tiles leave SMs idle
    assert cut > 100


def test_pieces_of_k_for_few_rows():
    for M, N, K in SIZES:
        pieces = rules.choose_k_splits(M, N, K)
        assert 1 <= pieces <= 16, (M, N, K, pieces)
        if pieces > 1:
            assert K // 256 >= pieces                            # a piece keeps at least 256 elements of k


def test_the_pair_rules_exclude_each_other():
    for M, N, K in SIZES:
        whole, halves = rules.use_pair(M, N, K), rules.use_pair_halves(M, N, K)
        assert not (whole and halves), (M, N, K)
        if halves:
            assert pieces_are_whole(K, 2) and N % 4 == 0 and M >= 1536
        if whole:
            assert N % 8 == 0 and -(-M // 256) * -(-N // 256) >= 44


def test_the_sizes_the_rules_were_measured_at():
    """Qwen2.5-0.5B: the down projection (N=896, K=4864) and the output projection (N=896, K=896)."""
    assert rules.choose_tile_k_splits(64, 896, 4864) == 8
    assert rules.choose_tile_k_splits(512, 896, 896) == 4            # 4 planes of 1.8 MB
    assert rules.choose_tile_k_splits(2048, 896, 4864) == 1          # planes of 7.3 MB: not on lone CTAs
    assert rules.use_pair_halves(2048, 896, 4864) and not rules.use_pair(2048, 896, 4864)
    assert rules.use_pair(4096, 896, 4864) and not rules.use_pair_halves(4096, 896, 4864)
    assert not rules.use_pair(2048, 896, 896) and not rules.use_pair_halves(2048, 1152, 896)
