"""Parity check that the multi-GPU benchmarks run inside their own processes before they time anything."""


def tp_parity(stack, make_ref, prompt, rank, dev, n_tokens=32):
    """Parity of the sharded stack inside the bench process: the first `n_tokens` greedy tokens of the tensor-parallel
    stack against the same tokens of an un-sharded decode stack (`make_ref()`, called on rank 0 only, builds it from
    the same seeded weights), then
    both fed the un-sharded run's sequence token by token: every position's arg-max must agree, or the un-sharded
    logits must hold the two candidates within 1e-2 or two rounding steps of the 16-bit type the logits are stored in,
    whichever is larger (the sharded fp32 sums round in another order).

    Mixture-of-experts stacks (those with `router_state()`) are also compared layer by layer on their routing, the one
    discontinuous step of the model: where the sharded run picks another expert than the un-sharded one, the first
    such layer of the step is looked at, and the pick counts as a near-tie when the un-sharded router logits of the two
    experts are within two rounding steps of the 16-bit type (the logits are stored in it). A position whose token
    differs in a step with such a flip is reported as explained by routing."""
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
    moe = hasattr(stack, "router_state")
    route = {"steps": 0, "steps_with_flip": 0, "flips_at_near_tie": 0, "flips_elsewhere": 0}
    explained = 0
    ulp = 2.0 ** -7 if stack.dtype == torch.bfloat16 else 2.0 ** -10
    for t in range(seq.shape[1]):
        tok = seq[:, t].contiguous()
        stack.set_tokens(tok)
        stack.step()
        if ref is not None:
            ref.set_tokens(tok)
            ref.step()
        if ref is None:
            continue
        flip_near_tie = False
        if moe:
            rl, ri = ref.router_state()
            _, si = stack.router_state()
            rl, ri, si = rl.cpu(), ri.cpu(), si.cpu()
            route["steps"] += 1
            differ = (ri != si).any(dim=1).nonzero()
            if differ.numel():
                l = int(differ[0])
                pa, pb = int(ri[l, 0]), int(si[l, 0])
                gap = abs(float(rl[l, pa] - rl[l, pb]))
                flip_near_tie = gap <= 2 * ulp * max(abs(float(rl[l, pa])), abs(float(rl[l, pb])), 1e-6)
                route["steps_with_flip"] += 1
                route["flips_at_near_tie" if flip_near_tie else "flips_elsewhere"] += 1
        if t < T - 1:
            continue
        a, b = int(stack.next_tokens()[0].item()), int(ref.next_tokens()[0].item())
        if a == b:
            agree += 1
            continue
        if flip_near_tie:
            explained += 1
            continue
        lg = ref.logits()[0].float()
        margin = float((lg[b] - lg[a]).item())
        first_margin = margin if first_margin is None else first_margin
        worst = max(worst, margin)
        # the logits are stored in the 16-bit type: two rounding steps at their magnitude, or 1e-2 where that is less
        step = 2 * ulp * max(abs(float(lg[a])), abs(float(lg[b])))
        near_ties += 1 if 0 <= margin <= max(1e-2, step) else 0
    torch.cuda.synchronize()
    del ref
    out = {"against": "un-sharded decode stack on rank 0, same seeded weights", "tokens_checked": n_tokens,
           "equal_prefix": equal_prefix, "first_margin": first_margin,
           "teacher_forced": {"positions": n_tokens, "same_token": agree, "near_tie_flips": near_ties,
                              "other_mismatches": n_tokens - agree - near_ties - explained, "worst_margin": worst}}
    if moe:
        out["teacher_forced"]["explained_by_routing_near_tie"] = explained
        out["routing"] = route
    return out
