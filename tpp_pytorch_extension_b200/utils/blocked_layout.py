"""The blocked weight layout of the reference (src/tpp_pytorch_extension/utils/blocked_layout.py:28-91 with the
blocking FixLinear attaches, llm_common.py:468-490), for the one case the quantized path uses."""
import torch


def block_weight(w, bk=16, bc=64, vnni=2):
    """W[N, K] -> [N/bk, K/bc, bc/vnni, bk, vnni] (view [N/bk, bk, K/bc, bc/vnni, vnni], permute [0,2,3,1,4])."""
    N, K = w.shape
    if N % bk or K % bc:
        raise ValueError(f"Blocking factor doesn't divide dim evenly shape = {tuple(w.shape)}, BF = {(bk, bc)}")
    return w.view(N // bk, bk, K // bc, bc // vnni, vnni).permute(0, 2, 3, 1, 4).contiguous()


def unblock_weight(wb):
    K1, C1, C2, K2, C3 = wb.shape
    return wb.permute(0, 3, 1, 2, 4).contiguous().view(K1 * K2, C1 * C2 * C3)
