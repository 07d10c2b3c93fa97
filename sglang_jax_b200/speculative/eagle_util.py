"""Token-tree construction and verification for EAGLE-style speculative decoding.

Everything here is batched tensor code that runs on whatever device the inputs live on;
the greedy verifier dispatches to the sm_100a kernel when one is available.

Node numbering.  The root (the last verified token) is node 0.  Draft step 0 contributes
`topk` depth-1 candidates (ids 1..k); every later step s contributes `k*k` candidates of
depth s+1 (ids `1 + k + (s-1)*k*k + branch*k + choice`).  A parent always has a smaller id
than its children, so "sorted by id" is a topological order.

Reference: `python/sgl_jax/srt/speculative/eagle_util.py` (tree build),
`python/sgl_jax/srt/kernels/speculative/{build_eagle_tree_structure,verify_tree_greedy,
tree_speculative_sampling_target_only}_kernel.py`.
"""

from __future__ import annotations

import torch


def select_top_k_branches(step: int, topk: int, branch_scores: torch.Tensor | None, probs: torch.Tensor,
                          node_base: int):
    """Grow the tree by one level.

    `probs [B, k_prev, V]` are the draft distributions of the current branches
    (`k_prev = 1` at step 0), `branch_scores [B, k_prev]` their cumulative scores.
    Returns the level's candidates `(cand_tokens, cand_scores, cand_parent_branch)`, each
    `[B, k_prev*k]`, and the `k` best of them `(sel, )` as indices into the candidates."""
    B, kp, V = probs.shape
    p, idx = torch.topk(probs, topk, dim=-1)                   # [B, kp, k]
    if branch_scores is None:
        scores = p
    else:
        scores = p * branch_scores.unsqueeze(-1)
    cand_tokens = idx.reshape(B, kp * topk)
    cand_scores = scores.reshape(B, kp * topk)
    cand_branch = torch.arange(kp, device=probs.device).repeat_interleave(topk).expand(B, -1)
    if kp * topk == topk:
        sel = torch.arange(topk, device=probs.device).expand(B, -1)
    else:
        sel = torch.topk(cand_scores, topk, dim=-1).indices
        sel = torch.sort(sel, dim=-1).values
    return cand_tokens, cand_scores, cand_branch, sel


def build_tree(verified_id: torch.Tensor, cand_tokens: torch.Tensor, cand_scores: torch.Tensor,
               cand_parent: torch.Tensor, num_draft_tokens: int, max_depth: int):
    """Pick the `num_draft_tokens - 1` best candidates and lay the tree out.

    `cand_* [B, C]`; `cand_parent` holds parent *node ids* (0 = root).
    Returns `tokens [B, n]` (node 0 = verified id), `parent [B, n]` (tree index of the parent,
    -1 for the root, -2 for a node whose parent was not selected), `depth [B, n]`,
    `mask [B, n, n]` (bool; row i sees its ancestors and itself) and `sel [B, n-1]`
    (candidate index of every non-root tree node)."""
    B, C = cand_tokens.shape
    n_sel = min(num_draft_tokens - 1, C)
    dev = cand_tokens.device
    # stable: on score ties a parent (smaller index) stays ahead of its children
    order = torch.sort(cand_scores, dim=-1, descending=True, stable=True).indices[:, :n_sel]
    sel = torch.sort(order, dim=-1).values                         # ascending node id
    n = n_sel + 1
    tokens = torch.cat([verified_id.view(B, 1).to(cand_tokens.dtype), cand_tokens.gather(1, sel)], dim=1)
    node_ids = torch.cat([torch.zeros(B, 1, dtype=torch.long, device=dev), sel + 1], dim=1)      # [B, n]
    inv = torch.full((B, C + 1), -2, dtype=torch.long, device=dev)
    inv.scatter_(1, node_ids, torch.arange(n, device=dev).expand(B, -1))
    parent_node = torch.cat([torch.zeros(B, 1, dtype=torch.long, device=dev), cand_parent.gather(1, sel)], dim=1)
    parent = inv.gather(1, parent_node)
    parent[:, 0] = -1
    depth = torch.zeros(B, n, dtype=torch.long, device=dev)
    mask = torch.eye(n, dtype=torch.bool, device=dev).unsqueeze(0).repeat(B, 1, 1)
    cur = parent.clone()
    rows = torch.arange(n, device=dev).expand(B, -1)
    bidx = torch.arange(B, device=dev).view(B, 1).expand(-1, n)
    for _ in range(max_depth):
        ok = cur >= 0
        depth += ok.long()
        c = cur.clamp_min(0)
        mask[bidx[ok], rows[ok], c[ok]] = True
        nxt = parent.gather(1, c)
        cur = torch.where(ok, nxt, cur)
    orphan = (parent == -2)
    if orphan.any():
        # a node whose ancestor chain is broken can never be accepted; park it at depth 1
        depth = torch.where(orphan, torch.ones_like(depth), depth)
    return tokens, parent, depth, mask, sel


def verify_tree_greedy(tokens: torch.Tensor, parent: torch.Tensor, target_ids: torch.Tensor, max_depth: int):
    """Walk the tree from the root following the target's argmax.

    Returns `accept_len [B]` (number of accepted draft tokens), `path [B, max_depth+1]`
    (tree indices of the accepted chain starting with the root, -1 padded) and
    `bonus [B]` (the target's token after the last accepted node)."""
    B, n = tokens.shape
    dev = tokens.device
    if tokens.is_cuda:
        from .. import ops
        if ops.use_native(tokens):
            return ops._native().verify_tree_greedy(tokens, parent, target_ids, max_depth)
    cur = torch.zeros(B, dtype=torch.long, device=dev)
    alive = torch.ones(B, dtype=torch.bool, device=dev)
    accept = torch.zeros(B, dtype=torch.long, device=dev)
    path = torch.full((B, max_depth + 1), -1, dtype=torch.long, device=dev)
    path[:, 0] = 0
    tgt = target_ids.long()
    for d in range(1, max_depth + 1):
        want = tgt.gather(1, cur.view(B, 1))
        match = (parent == cur.view(B, 1)) & (tokens.long() == want) & alive.view(B, 1)
        match[:, 0] = False
        has = match.any(dim=1)
        nxt = match.float().argmax(dim=1)
        cur = torch.where(has, nxt, cur)
        alive &= has
        accept += has.long()
        path[:, d] = torch.where(has, nxt, torch.full_like(nxt, -1))
    bonus = tgt.gather(1, cur.view(B, 1)).squeeze(1)
    return accept, path, bonus


def tree_speculative_sampling_target_only(tokens: torch.Tensor, parent: torch.Tensor, target_probs: torch.Tensor,
                                          coins: torch.Tensor, final_coins: torch.Tensor, max_depth: int,
                                          threshold_single: float = 1.0, threshold_acc: float = 1.0):
    """Stochastic verification when the draft is deterministic (top-k proposals).

    At every level one uniform coin is compared against the cumulative target probability
    of the children in index order: child i is accepted when the coin falls inside its
    interval, which happens with probability `p_target(child i)`.  When no child is
    accepted the bonus token is drawn from the target distribution with the rejected
    children removed.  With both thresholds at 1 the output distribution equals plain
    sampling from the target.  `target_probs [B, n, V]`, `coins [B, max_depth+1]`,
    `final_coins [B]`."""
    B, n = tokens.shape
    dev = tokens.device
    tok = tokens.long()
    par = parent.clamp_min(0)
    bidx = torch.arange(B, device=dev).view(B, 1).expand(-1, n)
    # probability the *parent's* distribution assigns to each node's token
    ptok = target_probs[bidx, par, tok]                                # [B, n]
    cur = torch.zeros(B, dtype=torch.long, device=dev)
    depth = torch.zeros(B, dtype=torch.long, device=dev)
    acc = torch.zeros(B, dtype=target_probs.dtype, device=dev)
    accept = torch.zeros(B, dtype=torch.long, device=dev)
    path = torch.full((B, max_depth + 1), -1, dtype=torch.long, device=dev)
    path[:, 0] = 0
    ar = torch.arange(B, device=dev)
    for i in range(1, n):
        is_child = parent[:, i] == cur
        p_i = ptok[:, i]
        acc_new = acc + p_i
        coin = coins.gather(1, depth.clamp_max(max_depth).view(B, 1)).squeeze(1)
        ok = is_child & ((coin <= acc_new / threshold_acc) | (p_i >= threshold_single)) & (depth < max_depth)
        acc = torch.where(is_child & ~ok, acc_new, acc)
        # move down
        depth = torch.where(ok, depth + 1, depth)
        path[ar[ok], depth[ok]] = i
        cur = torch.where(ok, torch.full_like(cur, i), cur)
        acc = torch.where(ok, torch.zeros_like(acc), acc)
        accept += ok.long()
    # residual distribution at the stopping node: children of `cur` were all rejected
    resid = target_probs[ar, cur].clone()                              # [B, V]
    rejected = (parent == cur.view(B, 1))
    rejected[:, 0] = False
    rb, ri = rejected.nonzero(as_tuple=True)
    resid[rb, tok[rb, ri]] = 0
    s = resid.sum(dim=-1, keepdim=True)
    resid = torch.where(s > 0, resid / s.clamp_min(1e-20), target_probs[ar, cur])
    cdf = resid.cumsum(dim=-1)
    bonus = torch.searchsorted(cdf, (final_coins.view(B, 1).to(cdf.dtype) * cdf[:, -1:]).contiguous()).squeeze(1)
    bonus = bonus.clamp_max(resid.shape[-1] - 1)
    return accept, path, bonus
