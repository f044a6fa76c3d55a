"""Helpers shared by the GPU parity tests of the decode stack."""
import torch

from oracle import decode_oracle as oracle


def to_cuda(w):
    return {k: ([t.cuda() for t in v] if isinstance(v, list) else v.cuda()) for k, v in w.items()}


def check_greedy_tokens(stack, w_cpu, cfg, prompt, want, max_T, use_graph, near_tie=1e-2, label=""):
    """Greedy decoding of `stack` against the oracle's tokens `want` [1, n] for `prompt` [1, T].

    Identical tokens pass. Otherwise the stack is run again teacher-forced on the oracle's own sequence and EVERY
    one of the n positions is checked: its arg-max equals the oracle's token, or the oracle's logits at that position
    hold the two candidates within `near_tie` of each other (a summation-order difference can flip such a pair; any
    other difference is a bug). Returns the number of leading tokens of the free run that equal the oracle's."""
    n = want.shape[1]
    got = stack.greedy(prompt, n, use_graph=use_graph).cpu()
    same = int((got[0] == want[0]).long().cumprod(0).sum().item())
    if same == n:
        return same
    T = prompt.shape[1]
    ref = oracle.LlamaOracle(w_cpu, cfg, max_T=max_T)
    seq = torch.cat((prompt, want[:, :-1]), dim=1)
    stack.reset(0)
    flips = []
    for t in range(seq.shape[1]):
        logits = ref.forward(seq[:, t:t + 1])[0]
        stack.set_tokens(seq[:, t].contiguous())
        stack.step()
        if t < T - 1:
            continue
        i = t - (T - 1)
        tok = int(stack.next_tokens()[0].item())
        wt = int(want[0, i])
        if tok != wt:
            margin = (logits[wt] - logits[tok]).item()
            assert 0 <= margin < near_tie, (f"{label}: position {i}: stack picks {tok}, oracle {wt}, oracle logit "
                                            f"margin {margin} is no near-tie; free run equal for {same} tokens")
            flips.append(i)
    return same


def reference_gateup_pack(gate_q, gate_scales_min, up_q, up_scales_min):
    """Separate per-group 8-bit gate / up tensors -> the reference's pack: bytes [I, H, 2] (gate, up interleaved
    element by element) and {scale, min} pairs [I * G, 2, 2] (gate pair, up pair), the layout built by
    muillm/modules/quantized/int8gateupdownmlp.py:211-230 (`_pack_gateup_weights`, `_pack_gateup_linears`)."""
    import torch

    pack = torch.stack([gate_q, up_q], dim=-1).contiguous()
    sm = torch.stack([gate_scales_min.reshape(-1, 2), up_scales_min.reshape(-1, 2)], dim=1).contiguous()
    return pack, sm

