"""Generates ``c3_decode_128.npz``: the oracle's greedy continuation on the Llama-3.2-1B-shaped
benchmark configuration (random Q4_K_M-mix weights, f16 KV cache prefilled with 1024 seeded positions,
a seeded 16-token prompt processed token by token, then 128 greedy tokens with no penalties:
crates/ullm-model/src/lib.rs:807-969 with argmax crates/ullm-model/src/sample.rs:125-133).

Stored per generated step: the token, the runner-up, and the gap between their logits divided by the
largest |logit| of the step (the quantity the 1e-3 logit tolerance is stated in), so that a GPU test
can tell a real divergence from a near-tie.  Run:  python tests/golden/make_c3_decode.py  (about a
minute of CPU time; the oracle must be built).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import oracle  # noqa: E402
from ullm_b200 import synth  # noqa: E402

N_PRE, N_PROMPT, N_GEN = 1024, 16, 128


def oracle_model(m, kv_f16):
    mk = lambda t: oracle.Weight(t[0], t[1], t[2], t[3])
    layers = [{k: (mk(v) if isinstance(v, tuple) else v) for k, v in l.items()} for l in m["layers"]]
    return oracle.LlamaModel(m["params"], mk(m["tok_embd"]), mk(m["output"]), m["final_norm"], layers, kv_f16)


def main():
    p = dict(synth.LLAMA_1B)
    m = synth.gen_llama_model(p, synth.seed_for(3, 0))
    k, v = synth.gen_kv_prefill(p, N_PRE, synth.seed_for(3, 1))
    prompt = synth.rand_ints(synth.seed_for(3, 2), N_PROMPT, 0, p["vocab"] - 1)
    om = oracle_model(m, True)
    om.key_cache[:, :N_PRE] = k
    om.val_cache[:, :N_PRE] = v
    for i, t in enumerate(prompt):
        lg = om.forward(int(t), N_PRE + i)
    tokens, second, gap = [], [], []
    first = oracle.argmax(lg)
    t = first
    for i in range(N_GEN):
        lg = om.forward(t, N_PRE + N_PROMPT + i)
        order = np.argpartition(lg, -2)[-2:]
        a, b = (order[1], order[0]) if lg[order[1]] >= lg[order[0]] else (order[0], order[1])
        t = oracle.argmax(lg)
        assert t == int(a) or lg[t] == lg[a]
        tokens.append(t), second.append(int(b))
        gap.append(float(lg[t] - lg[b]) / float(np.max(np.abs(lg))))
    np.savez(os.path.join(HERE, "c3_decode_128.npz"), prompt=np.asarray(prompt, np.uint32), first=np.uint32(first),
             tokens=np.asarray(tokens, np.uint32), second=np.asarray(second, np.uint32), rel_gap=np.asarray(gap, np.float32))
    print("first", first, "tokens", tokens[:8], "min rel gap", min(gap))


if __name__ == "__main__":
    main()
