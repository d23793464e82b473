"""bfloat16 matrix products, 32-bit accumulation: chooses the kernel by the
number of rows.  Few rows (decoding) are bound by reading the weights once and
go to the framework's streaming kernel; many rows go to the tensor cores."""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..kernels import ops

# TOKB200_STREAM=0 keeps the vocabulary projection of few rows on the kernel for single products
_STREAM = os.environ.get("TOKB200_STREAM", "1") != "0"

_sm_count = None


def sm_count() -> int:
    """SMs of the current device (148 on a B200; that figure where no device is visible, so
    that the rules below can be read on a machine without one)."""
    global _sm_count
    if _sm_count is None:
        try:
            _sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count \
                if torch.cuda.is_available() else 148
        except Exception:
            _sm_count = 148
    return _sm_count


def _target_blocks() -> int:
    """Blocks wanted in flight before a product with few weight rows is also cut along k."""
    return 2 * sm_count()


def choose_k_splits(M: int, N: int, K: int) -> int:
    """How many pieces along k a small-M product is cut into (1: none)."""
    tiles = (N + 15) // 16
    blocks = (tiles + 1) // 2 if tiles >= 1024 else tiles
    if blocks >= _target_blocks() // 2:
        return 1
    return max(1, min(-(-_target_blocks() // blocks), K // 256, 16))


def choose_tile_k_splits(M: int, N: int, K: int) -> int:
    """Pieces of k for a many-row product whose output tiles (128 x 128) are too few for the
    device: about one unit of work per SM, at least two 64-element blocks of k a piece."""
    tiles = -(-M // 128) * -(-N // 128)
    k_blocks = -(-K // 64)
    sms = sm_count()
    if tiles * 2 > sms or N % 4 or k_blocks < 4:
        return 1
    want = min(sms // tiles, k_blocks // 2, 8)      # more pieces cost the consumer more than they save here
    # the consumer reads every plane: beyond 8 MB of partial sums adding them costs more than the
    # idle SMs did (a step of 512 rows: 1.98 -> 1.81 ms with at most 4 planes of 1.8 MB)
    plane = M * N * 4
    want = 1 if plane > 4_000_000 else max(1, min(want, 8_000_000 // plane))
    per = -(-k_blocks // max(want, 1))
    return -(-k_blocks // per)


def use_pair(M: int, N: int, K: int) -> bool:
    """Many rows, a long k and enough tiles of 256 x 256 for most of a device's 74 pairs of SMs
    (the down projection from 2,816 rows on, where tiles of 128 x 128 need a second round of
    CTAs and take 48 us at 3,072 rows): the product goes to pairs of CTAs, each loading half of
    the weight tile."""
    return ops._PAIR and K >= 2048 and N % 8 == 0 and -(-M // 256) * -(-N // 256) >= (sm_count() // 2) * 3 // 5


def use_pair_halves(M: int, N: int, K: int) -> bool:
    """Between 1,536 rows and half the pairs' worth of tiles (the down projection of a portion of
    2,048 tokens: 32 tiles): the pair form with k cut in two, float32 partial sums for a consumer
    that adds them (product 25.2 -> 22.1 us, the norm behind it 3.6 -> 3.9 us)."""
    return ops._PAIR and M >= 1536 and K >= 2048 and N % 4 == 0 and \
        -(-M // 256) * -(-N // 256) <= sm_count() // 4


LIBRARY_ROWS = 256      # from here on every plain product goes to the vendor library unless TOKB200_GEMM=own


def use_tcgen05(M: int, N: int, K: int, cut_along_k: bool = False) -> bool:
    """Which plain products (no epilogue of the framework's own) go to the framework's tcgen05
    kernel: those of up to 64 rows, and from 65 to LIBRARY_ROWS - 1 rows the long-k products cut along k.  With more rows the vendor library's product
    leads it at the layer sizes measured (a captured chain of products, us, library / own best
    form): 512 rows, hidden 896: q/k/v 4.4 / 6.7, output 3.9 / 6.1, down 9.0 / 10.3; 2,048 rows:
    6.3 / 8.3, 5.7 / 8.2, 14.5 / 22.0; hidden 1,536, 512 rows: 6.0 / 8.3, 5.1 / 7.3, 15.6 / 20.4;
    hidden 3,584, 512 rows: 14.8 / 30.4, 12.1 / 30.3, 59.5 / 172.7; 2,048 rows: 52.7 / 50.9,
    43.3 / 45.5, 192.6 / 211.7.  The own kernel's tiles of 128 x 128 keep five stages of 32 KB in
    flight per multiprocessor, which at the latency of a load from L2 feeds the tensor core at
    about 0.4 of its rate (tensor pipe 45 % on the down projection); only its 256 x 256 tiles on
    pairs of CTAs (the gate/up product with its activation, which stays the framework's own at
    every row count) move few enough bytes per instruction.  TOKB200_GEMM=own keeps every
    product on the own kernels, TOKB200_GEMM=library sends all plain many-row products to the
    library; sizes the kernel does not take (K not a multiple of 8) go there as well."""
    choice = os.environ.get("TOKB200_GEMM", "")
    if choice == "library" or not ops.gemm_tcgen05_supported(M, N, K):
        return False
    if choice == "own" or M <= 64:
        return True
    if M < LIBRARY_ROWS:
        # 65 to 255 rows: the own kernel's floor is 5 to 8 us where the library's product takes 3.5
        # (q/k/v 1152 x 896 at 128 rows: 8.5 against 3.6, output 5.4 against 3.6); only the long-k
        # product cut along k into partial sums leads it (down 896 x 4864: 7.6 against 8.5)
        return cut_along_k and K >= 4 * N
    return False


STREAM_WHOLE_ROW = 1024     # the longest row (elements) that the ring-streaming kernel copies in one piece


def linear_bf16(a: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                out_dtype: torch.dtype, partials_ok: bool = False) -> torch.Tensor:
    """a[M,K] weight[N,K]^T (+ bias float32) as bfloat16 or float32 [M,N]; with
    `partials_ok` the result may be float32 partial sums [S,M,N] instead."""
    M, K = a.shape
    N = weight.shape[0]
    # few rows: the streaming kernel; up to 64 rows it also keeps the narrow matrices,
    # whose few tiles would leave most SMs of the tile kernel idle
    # few rows and a weight of many rows (the vocabulary projection): one block an SM streams
    # its run of the weight through a shared-memory ring.  Only where a copy brings a whole row
    # (K up to STREAM_WHOLE_ROW): the copy engine takes a fixed time per copy, so that pieces of
    # 1 KB stream at 3.2 TB/s where whole rows of 1.8 KB reach 5.4 and the kernel below 5.7 to 6.7.
    if _STREAM and M <= ops.SMALL_M_ROWS and K <= STREAM_WHOLE_ROW and N >= 16 * sm_count() * 4 and \
            ops.linear_stream_supported(M, N, K):
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        ops.linear_stream(a, weight, bias, out)
        return out
    if out_dtype == torch.bfloat16 and use_tcgen05(M, N, K) and use_pair(M, N, K):
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        ops.gemm_tcgen05_pair(a, weight, bias, out, ops.PAIR_PLAIN)
        return out
    if partials_ok and bias is None and use_tcgen05(M, N, K) and use_pair_halves(M, N, K):
        out = torch.empty((2, M, N), dtype=torch.float32, device=a.device)
        ops.gemm_tcgen05_pair(a, weight, None, out, ops.PAIR_PARTIALS)
        return out
    tiles_cut = 1
    if ops._RING and partials_ok and bias is None and ops.SMALL_M_ROWS < M <= ops.RING_MAX_ROWS and N <= 2048:
        # 17 to 32 rows and a narrow output whose consumer takes partial sums (the output and down
        # projections of a model up to hidden 2,048): the ring kernel leads the tensor-core tiles cut
        # along k (hidden 896: down 7.1 -> 5.2 to 5.8 us, output 4.9 -> 3.8 to 4.5; hidden 1,536: 11.5 ->
        # 10.2 to 11.3, 5.5 -> 4.3; at hidden 3,584 it does not)
        splits = ops.linear_ring_splits(M, N, K, sm_count())
        if splits:
            out = torch.empty((splits, M, N), dtype=torch.float32, device=a.device) if splits > 1 else \
                torch.empty((M, N), dtype=out_dtype, device=a.device)
            ops.linear_ring(a, weight, None, out, splits)
            return out
    if partials_ok and bias is None and M > ops.SMALL_M_ROWS and use_tcgen05(M, N, K, cut_along_k=True):
        tiles_cut = choose_tile_k_splits(M, N, K)
    if tiles_cut > 1:
        # few output tiles (a narrow matrix, a few dozen rows): pieces of k over all SMs
        out = torch.empty((tiles_cut, M, N), dtype=torch.float32, device=a.device)
        ops.gemm_tcgen05_partials(a, weight, out)
        return out
    if ops._RING and M <= ops.SMALL_M_ROWS and N * K >= ops.RING_ELEMENTS:
        # few rows and a large weight (a wide model's matrices, its vocabulary projection): one block a
        # multiprocessor streams it through rings in shared memory (`linear_ring.cu`)
        splits = ops.linear_ring_splits(M, N, K, sm_count()) if (partials_ok and bias is None) else \
            (1 if ops.linear_ring_supported(M, N, K, 1) else 0)
        if splits:
            out = torch.empty((splits, M, N), dtype=torch.float32, device=a.device) if splits > 1 else \
                torch.empty((M, N), dtype=out_dtype, device=a.device)
            ops.linear_ring(a, weight, bias, out, splits)
            return out
    if ops.linear_small_m_supported(M, K) and (M <= ops.SMALL_M_ROWS or N < 4096):
        splits = choose_k_splits(M, N, K) if (partials_ok and bias is None) else 1
        if splits > 1:
            out = torch.empty((splits, M, N), dtype=torch.float32, device=a.device)
        else:
            out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        ops.linear_small_m(a, weight, bias, out, splits)
        return out
    if use_tcgen05(M, N, K):
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        ops.gemm_tcgen05(a, weight, bias, out)
        return out
    # the vendor library, for the shapes where it still leads the kernel above
    if out_dtype == torch.bfloat16:
        out = torch.mm(a, weight.t())
    else:
        out = torch.mm(a, weight.t(), out_dtype=torch.float32)
    if bias is not None:
        out.add_(bias.to(out.dtype) if out.dtype != torch.float32 else bias)
    return out
