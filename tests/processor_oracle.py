"""The processors' dataflow restated with plain torch + the CPU oracle (test infrastructure):
what the reference's WanAttn_SAPAttn_Processor / Hunyuan_SAPAttn_Processor2_0 compute for the
fixture cases of tests/golden_util.py, step by step, from the recorded initial indices."""
import os

import torch

from oracle import svoo_oracle as O
from svoo_b200.sparsity import SparsityLookup
from tests import golden_util as gu


def wan_steps(z):
    """Runs the four steps of the WAN_PROC case through the oracle's processor
    (oracle/wan_processor.py), replaying the recorded initial indices.  Yields
    (step, sparse?, out [S, dim] bf16, aux dict or None)."""
    from oracle.wan_processor import OracleWanProcessor
    P = gu.WAN_PROC
    H = P["heads"]
    T, Hh, W = P["grid"]
    N = T * Hh * W
    cls = type("OracleWanProcessorCase", (OracleWanProcessor,), {})
    gu.configure_wan_processor(cls, SparsityLookup(os.path.join(gu.GOLDEN, "processor_wan_density.csv")))
    attn = gu.make_attn(31, H)
    cos, sin = gu.rotary_tables(32, N)
    proc = cls(0)
    with torch.no_grad():
        for step, tval in P["steps"]:
            hidden = gu.wan_step_hidden(step)
            proc._step_from_callback = step
            qi = torch.from_numpy(z[f"q_init_{step}"]).long()
            ki = torch.from_numpy(z[f"k_init_{step}"]).long()
            proc.draw_init_indices = lambda BH, n, qi=qi, ki=ki: (qi, ki)
            y = proc(attn, hidden, rotary_emb=(cos, sin), timestep=torch.tensor([tval]))
            yield step, proc.last_aux is not None, y[0], proc.last_aux


def hunyuan_qkv(attn, hidden, enc):
    """q, k, v [1,H,S,128] of a single-stream block without rotary tables
    (svoo/models/hunyuan10/attention.py:545-561)."""
    x = torch.cat([hidden, enc], dim=1)
    q, k, v = (t.unflatten(2, (attn.heads, -1)).transpose(1, 2).contiguous() for t in (attn.to_q(x), attn.to_k(x), attn.to_v(x)))
    return attn.norm_q(q), attn.norm_k(k), v


def hunyuan_step(z):
    """The HUN_PROC case through the oracle: (out [N, dim], out_enc [ctx, dim], aux)."""
    P = gu.HUN_PROC
    attn = gu.make_attn(41, P["heads"], joint=True)
    hidden, enc, mask = gu.hunyuan_inputs()
    with torch.no_grad():
        q, k, v = hunyuan_qkv(attn, hidden, enc)
        qi, ki = torch.from_numpy(z["q_init"]).long(), torch.from_numpy(z["k_init"]).long()
        o, aux = O.sparse_attention_layer(q, k, v, qi, ki, P["num_q"], P["num_k"], P["iter_init"], P["top_p"],
                                          float(P["min_kc_ratio"]), 0, P["context_length"], P["prompt_length"])
        y = o.transpose(1, 2).flatten(2, 3)
        ctx = P["context_length"]
        return attn.to_out[0](y[:, :-ctx])[0], y[0, -ctx:], aux
