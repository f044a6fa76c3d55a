"""Parity check that the multi-GPU benchmarks run inside their own processes before they time anything."""


def tp_parity(stack, make_ref, prompt, rank, dev, n_tokens=32):
    """Parity of the sharded stack inside the bench process: the first `n_tokens` greedy tokens of the tensor-parallel
    stack against the same tokens of an un-sharded decode stack (`make_ref()`, called on rank 0 only, builds it from
    the same seeded weights), then
    both fed the un-sharded run's sequence token by token: every position's arg-max must agree, or the un-sharded
    logits must hold the two candidates within 1e-2 (the sharded fp32 sums round in another order)."""
    import torch
    import torch.distributed as dist

    T = prompt.shape[1]
    ref_tokens = torch.zeros(1, n_tokens, dtype=torch.int64, device=dev)
    ref = None
    if rank == 0:
        ref = make_ref()
        ref_tokens.copy_(ref.greedy(prompt, n_tokens, use_graph=True))
    dist.broadcast(ref_tokens, 0)
    got = stack.greedy(prompt, n_tokens, use_graph=True)
    torch.cuda.synchronize()
    equal_prefix = int((got[0] == ref_tokens[0]).long().cumprod(0).sum().item())
    seq = torch.cat((prompt.to(dev), ref_tokens[:, :-1]), dim=1)
    stack.reset(0)
    if ref is not None:
        ref.reset(0)
    agree, near_ties, worst, first_margin = 0, 0, 0.0, None
    for t in range(seq.shape[1]):
        tok = seq[:, t].contiguous()
        stack.set_tokens(tok)
        stack.step()
        if ref is not None:
            ref.set_tokens(tok)
            ref.step()
        if t < T - 1 or ref is None:
            continue
        a, b = int(stack.next_tokens()[0].item()), int(ref.next_tokens()[0].item())
        if a == b:
            agree += 1
            continue
        lg = ref.logits()[0].float()
        margin = float((lg[b] - lg[a]).item())
        first_margin = margin if first_margin is None else first_margin
        worst = max(worst, margin)
        near_ties += 1 if 0 <= margin < 1e-2 else 0
    torch.cuda.synchronize()
    del ref
    return {"against": "un-sharded decode stack on rank 0, same seeded weights", "tokens_checked": n_tokens,
            "equal_prefix": equal_prefix, "first_margin": first_margin,
            "teacher_forced": {"positions": n_tokens, "same_token": agree, "near_tie_flips": near_ties,
                               "other_mismatches": n_tokens - agree - near_ties, "worst_margin": worst}}
