"""CPU restatement of the reference's mean-similarity block selection (flash_attn/utils/sparse_utils.py:376-441:
get_block_map_meansim; pooling and self-similarity :281-299 triton_bmm_pool_sim_simmean; map fill :336-347; causal block
mask :359-366).  TEST INFRASTRUCTURE ONLY: imported by tests/, never by the product path.

Parity unpinned: the reference's version runs Triton kernels and 16-bit torch ops on its own device; neither runs here,
and the reference's tests hold no vectors for it.  This file follows the reference's steps one by one but evaluates
step 2 in fp32 (the reference keeps its score, softmax and cumulative-sum tensors in the 16-bit input type, with
device-library-dependent rounding), and returns the decision margins so that a test can leave out the blocks whose
choice hangs on the last bits.
"""
import torch


def pool_sim_ref(x: torch.Tensor, block_size: int, simthreshd1: torch.Tensor):
    """x (B, H, N, D) 16-bit -> pooled (B, H, nb, D) in x.dtype, sim (B, H, nb) bool, value (B, H, nb) fp32 (the mean
    pairwise cosine similarity that is compared with simthreshd1[h]; NaN where the reference's is: blocks cut short by the
    end of the sequence, blocks holding a zero row).  sparse_utils.py:281-299."""
    B, H, N, D = x.shape
    nb = (N + block_size - 1) // block_size
    pooled = torch.zeros(B, H, nb, D, dtype=x.dtype)
    value = torch.zeros(B, H, nb, dtype=torch.float32)
    for i in range(nb):
        blk = x[:, :, i * block_size:(i + 1) * block_size].float()          # (B, H, rows, D)
        rows = blk.shape[2]
        pooled[:, :, i] = (blk.sum(dim=2) / rows).to(x.dtype)
        norm = blk.pow(2).sum(dim=-1, keepdim=True).sqrt()
        xh = (blk / norm).to(torch.float16).float()
        grams = xh @ xh.transpose(-1, -2)
        v = grams.sum(dim=(-1, -2)) / (rows * rows)
        if rows < block_size:                                               # padded rows: 0 / 0 in the reference
            v = torch.full_like(v, float("nan"))
        value[:, :, i] = v
    sim = value > simthreshd1.view(1, H, 1)                                 # NaN compares false
    return pooled, sim, value


def block_map_meansim_ref(q, k, is_causal=False, BLKQ=128, BLKK=64, simthreshd1=0.1, cdfthreshd=0.9, topk=None,
                          attention_sink=False):
    """q, k (B, H, N, D).  Returns (block_map (B, H, nq, nk) bool, margin (B, H, nq) fp32): margin = the smaller of the
    distance of the cumulative sums from cdfthreshd (inf with topk) and a tenth of the relative gap between the last
    kept and the first dropped probability; a test treats rows with a tiny margin as undecided."""
    assert (cdfthreshd is None) != (topk is None)
    B, H, _, D = q.shape
    f = lambda v: torch.full((H,), float(v)) if not torch.is_tensor(v) else v.float().reshape(-1).expand(H).clone()
    th1 = f(simthreshd1)
    pq, sq, _ = pool_sim_ref(q, BLKQ, th1)
    pk, sk, _ = pool_sim_ref(k, BLKK, th1)
    nq, nk = pq.shape[2], pk.shape[2]
    score = pq.float() @ pk.float().transpose(-1, -2) * (D ** -0.5)
    simk = sk.unsqueeze(-2).expand(-1, -1, nq, -1)
    simq = sq.unsqueeze(-1).expand(-1, -1, -1, nk)
    score = score.masked_fill(~simk, float("-inf"))
    causal = None
    if is_causal:
        qi = torch.arange(nq).view(-1, 1)
        kj = torch.arange(nk).view(1, -1)
        causal = kj * BLKK < (qi + 1) * BLKQ                                # sparse_utils.py:359-366
        score = score.masked_fill(~causal, float("-inf"))
    mx = score.max(dim=-1, keepdim=True).values
    e = torch.where(torch.isinf(mx), torch.zeros_like(score), (score - mx).exp())
    ssum = e.sum(dim=-1, keepdim=True)
    prob = torch.where(ssum > 0, e / ssum, torch.zeros_like(e))
    srt = torch.sort(prob, dim=-1, descending=True, stable=True)
    cdf = torch.cumsum(srt.values, dim=-1)
    if cdfthreshd is not None:
        thr = f(cdfthreshd).view(1, H, 1, 1)
        num = (cdf <= thr).sum(dim=-1)                                      # searchsorted(cdf, thr, right=True)
        margin = (cdf - thr).abs().min(dim=-1).values
    else:
        num = (f(topk) * nk).to(torch.int64).view(1, H, 1).expand(B, H, nq)
        margin = torch.full((B, H, nq), float("inf"))
    num = num.clamp(min=1, max=nk)
    # a tie (or near tie) between the last kept and the first dropped probability makes the choice arbitrary
    last = torch.gather(srt.values, -1, (num - 1).unsqueeze(-1)).squeeze(-1)
    nxt = torch.gather(srt.values, -1, num.clamp(max=nk - 1).unsqueeze(-1)).squeeze(-1)
    tie = torch.where(num < nk, (last - nxt).abs() / last.clamp_min(1e-30), torch.full_like(last, float("inf")))
    tie = torch.where((last == 0) & (nxt == 0), torch.full_like(tie, float("inf")), tie)   # both masked: same outcome
    margin = torch.minimum(margin, 0.1 * tie)     # a relative gap of 1e-4 at the cut counts like 1e-5 on the sums
    final = (~simk) | (~simq)
    rank = torch.argsort(srt.indices, dim=-1)                               # position of block j in the sorted order
    final = final | (rank < num.unsqueeze(-1))
    if is_causal:
        final = final & causal
    if attention_sink:
        final[..., 0] = True
    return final, margin
