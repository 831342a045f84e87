"""Generate the golden fixtures in this directory from the UNMODIFIED reference.

Run once, in a container that has the reference checkout (path in $SVOO_REFERENCE,
default: a directory `reference` beside this repository):

    python tests/golden/make_golden.py            # all fixtures (about 4 minutes)
    python tests/golden/make_golden.py layer_tiny_bf16   # just that one
    python tests/golden/make_golden.py processor_wan     # the processor fixtures: each in a process
    python tests/golden/make_golden.py processor_hunyuan # of its own (they configure class attributes)

The reference's hot path is Triton + torch.  Its Triton kernels are executed on
CPU tensors by the Triton interpreter (TRITON_INTERPRET=1); the wrappers'
`assert x.is_cuda` checks are satisfied by overriding the `is_cuda` property, so
every wrapper (co_cluster_tokens, permute_tensor_by_labels_triton,
apply_inverse_permutation_triton, dynamic_block_sparse_fwd_triton) and the pure
torch identify_dynamic_map run exactly as written.  Inputs are re-creatable from
seeds (svoo_b200.synth); a checksum of them is stored so that a drift of the RNG
is detected instead of silently invalidating the fixture.
"""
import os
import sys
import time

os.environ["TRITON_INTERPRET"] = "1"
HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("SVOO_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference"))
sys.path.insert(0, REF)
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import numpy as np
import torch

torch.Tensor.is_cuda = property(lambda self: True)

import svoo.co_clustering as ref_cc                      # noqa: E402
from svoo.kernels.triton import permute as ref_pm        # noqa: E402
from svoo.sparsity.lookup import SparsityLookup as RefLookup   # noqa: E402

from svoo_b200 import synth                              # noqa: E402


checksum = synth.tensor_checksum


def f32(t):
    return t.float().numpy()


def bf16_bits(t):
    """The bit patterns of a bf16 tensor as int16 (numpy has no bf16); golden_util.from_bf16_bits undoes it."""
    assert t.dtype == torch.bfloat16
    return t.contiguous().view(torch.int16).numpy()


def layer_case(name, cfg, iters, density, rows_kept=8, max_ratio=None):
    """Whole path through the reference for one small layer config."""
    t0 = time.time()
    q, k, v = synth.make_qkv(cfg)
    H, N, D = cfg.heads, cfg.n_video, 128
    q_idx, k_idx = synth.init_indices(cfg)
    torch.manual_seed(7)                                  # the reference draws from the global RNG
    ql, qc, qs, kl, kc, ks = ref_cc.co_cluster_tokens(q[0], k[0], cfg.num_q, cfg.num_k, max_iters=iters)
    # the draws above must be the ones synth.init_indices reproduces
    torch.manual_seed(7)
    assert torch.equal(torch.randint(0, N, (H, cfg.num_q)), q_idx)
    assert torch.equal(torch.randint(0, N, (H, cfg.num_k)), k_idx)
    # one-iteration run from the same init: not yet amplified by later iterations
    torch.manual_seed(7)
    ql1, qc1, qs1, kl1, kc1, ks1 = ref_cc.co_cluster_tokens(q[0], k[0], cfg.num_q, cfg.num_k, max_iters=1)

    qp, q_sorted = ref_pm.permute_tensor_by_labels_triton(q, ql, dim=2)
    kp, k_sorted = ref_pm.permute_tensor_by_labels_triton(k, kl, dim=2)
    vp, _ = ref_pm.permute_tensor_by_labels_triton(v, kl, dim=2, sorted_indices=k_sorted)
    args = dict(min_kc_ratio=density)
    if max_ratio is not None:
        args["max_kc_ratio"] = max_ratio
    dmap = ref_cc.identify_dynamic_map(qc.view(1, H, cfg.num_q, D), kc.view(1, H, cfg.num_k, D),
                                       qs.view(1, H, -1), ks.view(1, H, -1), cfg.top_p, **args)
    # The interpreter cannot run tl.dot on bf16 operands (numpy has no bf16), and the
    # attention kernel, unlike the clustering kernels, does not up-cast before its dots:
    # give it the same values as fp32.
    up = (lambda t: t.float()) if cfg.dtype == torch.bfloat16 else (lambda t: t)
    op = ref_cc.dynamic_block_sparse_fwd_triton(up(qp), up(kp), up(vp), dmap, qs.view(1, H, -1), ks.view(1, H, -1))
    out = ref_pm.apply_inverse_permutation_triton(op, q_sorted, dim=2)
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"),
        input_checksum=checksum(q, k, v),
        q_init_idx=q_idx.numpy().astype(np.int32), k_init_idx=k_idx.numpy().astype(np.int32),
        iters=np.array([iters]),
        qlabels=ql.numpy().astype(np.int16), klabels=kl.numpy().astype(np.int16),
        qcentroids=f32(qc), kcentroids=f32(kc), qsizes=qs.numpy(), ksizes=ks.numpy(),
        qlabels_it1=ql1.numpy().astype(np.int16), klabels_it1=kl1.numpy().astype(np.int16),
        qcentroids_it1=f32(qc1), kcentroids_it1=f32(kc1),
        q_sorted=q_sorted.numpy().astype(np.int32), k_sorted=k_sorted.numpy().astype(np.int32),
        min_kc_ratio=np.array(density if isinstance(density, list) else [density], dtype=np.float64),
        max_kc_ratio=np.array([-1.0] if max_ratio is None else
                              (max_ratio if isinstance(max_ratio, list) else [max_ratio]), dtype=np.float64),
        map_bits=np.packbits(dmap.numpy()), map_shape=np.array(dmap.shape),
        out_rows=f32(out[0, :, ::rows_kept]).astype(np.float32), rows_kept=np.array([rows_kept]),
        q_perm_rows=f32(qp[0, :, ::rows_kept * 4]),
    )
    print(f"{name}: {time.time() - t0:.1f}s  map density {dmap.float().mean():.3f}")


def map_case(name, H, QC, KC, dtype, p, min_ratio, max_ratio, seed):
    """identify_dynamic_map alone at production cluster counts."""
    g = torch.Generator("cpu").manual_seed(seed)
    base = torch.randn(H, 1, 128, generator=g)
    qc = (base + 0.7 * torch.randn(H, QC, 128, generator=g)).to(dtype)[None]
    kc = (base + 0.7 * torch.randn(H, KC, 128, generator=g)).to(dtype)[None]
    ks = torch.randint(0, 400, (1, H, KC), generator=g, dtype=torch.int32)
    ks[0, :, 3] = 0                                        # an empty key cluster
    qs = torch.randint(1, 900, (1, H, QC), generator=g, dtype=torch.int32)
    kw = {}
    if min_ratio is not None:
        kw["min_kc_ratio"] = min_ratio
    if max_ratio is not None:
        kw["max_kc_ratio"] = max_ratio
    dmap = ref_cc.identify_dynamic_map(qc, kc, qs, ks, p, **kw)
    def arr(r):
        if r is None:
            return np.array([-1.0])
        return np.array(r if isinstance(r, list) else [r], dtype=np.float64)
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"),
        seed=np.array([seed]), H=np.array([H]), QC=np.array([QC]), KC=np.array([KC]),
        is_bf16=np.array([dtype == torch.bfloat16]), p=np.array([p], dtype=np.float64),
        min_kc_ratio=arr(min_ratio), max_kc_ratio=arr(max_ratio),
        min_is_list=np.array([isinstance(min_ratio, list)]), max_is_list=np.array([isinstance(max_ratio, list)]),
        input_checksum=checksum(qc, kc, ks, qs),
        map_bits=np.packbits(dmap.numpy()), map_shape=np.array(dmap.shape),
    )
    print(f"{name}: kept per row mean {dmap.sum(-1).float().mean():.1f}")


def lookup_case():
    """SparsityLookup + per-head clipping on a small CSV in the shipped format."""
    import csv
    import tempfile
    g = torch.Generator("cpu").manual_seed(5)
    rows = []
    for step in (1, 2):
        for layer in range(3):
            for head in range(4):
                if (step, layer, head) == (2, 1, 3):
                    continue                               # a hole: that (step, layer) falls back
                rows.append((step, layer, head, float(torch.rand(1, generator=g)) * 0.6))
    path = os.path.join(HERE, "density_profile.csv")
    with open(path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["Step", "Layer", "Head", "Sparsity"])
        for r in rows:
            w.writerow([r[0], r[1], r[2], f"{r[3]:.6f}"])
    lk = RefLookup(path)
    got = np.array([[lk.get_sparsity_batch(s, l, 4) for l in range(3)] for s in (1, 2)])
    has = np.array([[lk.has_data_for_step_layer(s, l, 4) for l in range(3)] for s in (1, 2)])
    np.savez_compressed(os.path.join(HERE, "density_profile_expected.npz"), batch=got, has=has)
    print("lookup fixture written")


def producer_case(name, S, H, seed, eps=1e-6):
    """What the reference's processor hands to attention_core_logic: to_q/to_k/to_v, RMS norm over
    the whole projection (its Triton kernel, ENABLE_FAST_KERNEL=1), interleaved-pair rotary
    embedding, head transpose.  The processor module imports diffusers at its top, which is not
    installed here; the four names it imports are replaced by empty stand-ins (none of them is
    executed on this route), `torch.compile` is made the identity (the module compiles
    flex_attention at import), and `attention_core_logic` is replaced on the instance to capture
    its arguments.  Everything between is the reference's code, unmodified."""
    import types
    os.environ["ENABLE_FAST_KERNEL"] = "1"

    def mod(mname, **attrs):
        m = types.ModuleType(mname)
        m.__dict__.update(attrs)
        sys.modules.setdefault(mname, m)

    mod("diffusers")
    mod("diffusers.models")
    mod("diffusers.models.attention_processor", Attention=type("Attention", (torch.nn.Module,), {}))
    mod("diffusers.models.normalization", RMSNorm=type("RMSNorm", (torch.nn.Module,), {}))
    mod("diffusers.models.transformers")
    mod("diffusers.models.transformers.transformer_wan", _get_added_kv_projections=None, dispatch_attention_fn=None)
    real_compile = torch.compile
    torch.compile = lambda f=None, **kw: f
    try:
        import svoo.models.wan.attention as ref_attn
    finally:
        torch.compile = real_compile

    D = 128
    g = torch.Generator("cpu").manual_seed(seed)
    hidden = torch.randn(1, S, H * D, generator=g).bfloat16()
    attn = torch.nn.Module()
    for nm in ("to_q", "to_k", "to_v"):
        lin = torch.nn.Linear(H * D, H * D, bias=True)
        with torch.no_grad():
            lin.weight.copy_(torch.randn(H * D, H * D, generator=g) / (H * D) ** 0.5)
            lin.bias.copy_(torch.randn(H * D, generator=g) * 0.1)
        setattr(attn, nm, lin.bfloat16())
    for nm in ("norm_q", "norm_k"):
        nrm = torch.nn.Module()
        nrm.weight = torch.nn.Parameter((1.0 + 0.2 * torch.randn(H * D, generator=g)).bfloat16())
        nrm.eps = eps
        setattr(attn, nm, nrm)
    attn.heads = H
    attn.add_k_proj = None
    attn.to_out = torch.nn.ModuleList([torch.nn.Identity(), torch.nn.Identity()])
    # rotary tables in the layout the caller's rotary module produces: [1, S, 1, D] fp32
    ang = torch.rand(S, D // 2, generator=g) * 6.2831853
    cos = torch.cos(ang).repeat_interleave(2, dim=-1)[None, :, None, :].contiguous()
    sin = torch.sin(ang).repeat_interleave(2, dim=-1)[None, :, None, :].contiguous()

    proc = ref_attn.WanAttn_SAPAttn_Processor(0)
    proc.measure_attention_sparsity = False
    seen = {}

    def capture(query, key, value, timestep):
        seen.update(q=query, k=key, v=value)
        return torch.zeros(1, S, H * D, dtype=query.dtype)

    proc.attention_core_logic = capture
    with torch.no_grad():
        proc(attn, hidden, rotary_emb=(cos, sin), timestep=torch.tensor([5]))
        xq, xk, xv = attn.to_q(hidden), attn.to_k(hidden), attn.to_v(hidden)
    assert seen["q"].shape == (1, H, S, D) and seen["q"].is_contiguous()
    np.savez_compressed(os.path.join(HERE, name + ".npz"), xq=f32(xq), xk=f32(xk), xv=f32(xv),
                        wq=f32(attn.norm_q.weight.detach()), wk=f32(attn.norm_k.weight.detach()), eps=np.float32(eps),
                        cos=cos.numpy(), sin=sin.numpy(), q=f32(seen["q"]), k=f32(seen["k"]), v=f32(seen["v"]))
    print(name, "written")


def euclid_case(name="euclid_fp32"):
    """batch_kmeans_Euclid and euclid_assign_triton (svoo/co_clustering.py:335-541) on one small fp32
    problem (the interpreter cannot run the kernel's tl.dot on bf16 operands): 3 iterations from
    given initial centroids with tol = 0, so that the loop runs to max_iters."""
    from tests import golden_util as gu
    cfg = gu.EUCLID_CASE
    q, _, _ = synth.make_qkv(cfg)
    x = q[0]
    init = synth.init_indices(cfg)[0]
    c0 = torch.gather(x, 1, init[..., None].expand(-1, -1, 128))
    labels, cent, sizes, n_it = ref_cc.batch_kmeans_Euclid(x, cfg.num_q, max_iters=3, tol=0.0, init_centroids=c0.clone())
    x_sq = (x ** 2).sum(-1)
    one = ref_cc.euclid_assign_triton(x, c0, x_sq)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), input_checksum=checksum(x), labels=labels.numpy().astype(np.int16),
                        centroids=f32(cent), sizes=sizes.numpy().astype(np.int32), iters=np.array([n_it]),
                        labels_first_assign=one.numpy().astype(np.int16))
    print(name, "written:", n_it, "iterations")


def ear_case(name, cfg, settings):
    """The error-aware routing variant (svoo/co_clustering.py:1314-2050) on one small problem:
    value centroids (the Wan processor's _compute_value_centroids), error_estimation_triton,
    identify_dynamic_map_estimated for each (top_p, gamma, min_kc_ratio) of `settings`, and the
    centroid-compensation kernel _fused_qc_kernel_opt.  That kernel's wrapper obtains the token part
    (o, log2-sum-exp) from FlashInfer's CUDA code; here the token part is the exact masked softmax
    (oracle.ear_oracle.token_attention_with_lse), the kernel itself runs as written.
    For a bf16 case the interpreter cannot run tl.dot on bf16 operands: error_estimation_triton is
    given fp32 copies of its tensor arguments (the torch part of the selection sees bf16)."""
    from oracle import ear_oracle as E
    ref_wan, _ = _import_reference_processors()
    t0 = time.time()
    q, k, v = synth.make_qkv(cfg)
    H, N, D = cfg.heads, cfg.n_video, 128
    torch.manual_seed(7)
    ql, qc, qs, kl, kc, ks = ref_cc.co_cluster_tokens(q[0], k[0], cfg.num_q, cfg.num_k, max_iters=2)
    qp, q_sorted = ref_pm.permute_tensor_by_labels_triton(q, ql, dim=2)
    kp, k_sorted = ref_pm.permute_tensor_by_labels_triton(k, kl, dim=2)
    vp, _ = ref_pm.permute_tensor_by_labels_triton(v, kl, dim=2, sorted_indices=k_sorted)
    vc = ref_wan.WanAttn_SAPAttn_Processor._compute_value_centroids(v[0], kl, ks, cfg.num_k)
    qc4, kc4, vc4 = (t.view(1, H, -1, D) for t in (qc, kc, vc))
    qs3, ks3 = qs.view(1, H, -1), ks.view(1, H, -1)
    lowp = cfg.dtype == torch.bfloat16
    orig_est = ref_cc.error_estimation_triton
    if lowp:
        def est32(qcen, kcen, vcen, pk, pv, a, b, c_logits, *rest, **kw):
            return orig_est(qcen.float(), kcen.float(), vcen.float(), pk.float(), pv.float(), a, b, c_logits.float(), *rest, **kw)
        ref_cc.error_estimation_triton = est32
    store = dict(input_checksum=checksum(q, k, v), qlabels=ql.numpy().astype(np.int16), klabels=kl.numpy().astype(np.int16),
                 qcentroids=f32(qc), kcentroids=f32(kc), vcentroids=f32(vc), qsizes=qs.numpy(), ksizes=ks.numpy(),
                 settings=np.array([[s[0], s[1]] for s in settings], dtype=np.float64),
                 ratios=np.array([np.resize(np.asarray(s[2], dtype=np.float64), H) for s in settings]),
                 ratio_is_list=np.array([isinstance(s[2], list) for s in settings]))
    try:
        for n, (top_p, gamma, ratio) in enumerate(settings):
            clog = torch.einsum("bhqd,bhkd->bhqk", qc4, kc4) * (D ** -0.5)
            sc = ref_cc.error_estimation_triton(qc4, kc4, vc4, kp, vp, qs3, ks3, clog, gamma, 1e-8)
            m = ref_cc.identify_dynamic_map_estimated(qp, kp, vp, qs3, ks3, qc4, kc4, vc4, top_p, gamma=gamma, min_kc_ratio=ratio)
            store[f"scores_{n}"] = sc[0].numpy().astype(np.float32)
            store[f"map_bits_{n}"] = np.packbits(m[0].numpy())
            store["map_shape"] = np.array(m[0].shape)
            store[f"c_logits_{n}"] = f32(clog[0])
    finally:
        ref_cc.error_estimation_triton = orig_est
    # centroid compensation on the last map (fp32 copies for a bf16 case: tl.dot again)
    up = (lambda t: t.float()) if lowp else (lambda t: t)
    o_tok, lse2 = E.token_attention_with_lse(qp[0], kp[0], vp[0], m[0], qs, ks)
    o_flash = o_tok.to(q.dtype)                     # FlashInfer returns the tensors' dtype
    qf, o_in = up(qp[0]).contiguous(), up(o_flash).contiguous()
    kcf, vcf = up(kc).contiguous(), up(vc).contiguous()
    indptr = torch.zeros(1, H, cfg.num_q + 1, dtype=torch.int32)
    indptr[..., 1:] = torch.cumsum(qs3, -1)
    o_fin = torch.empty_like(qf)
    lse_fin = torch.empty(H, N, dtype=torch.float32)
    ref_cc._fused_qc_kernel_opt[(cfg.num_q, H)](
        Q=qf, K_centroids=kcf, V_centroids=vcf, block_mask_map=m, block_col_sz=ks3, O_flash=o_in, LSE_flash=lse2,
        QC_INDPTR=indptr, LSE_final=lse_fin, Out=o_fin,
        stride_qh=qf.stride(0), stride_qs=qf.stride(1), stride_qd=qf.stride(2),
        stride_ch=kcf.stride(0), stride_cn=kcf.stride(1), stride_cd=kcf.stride(2),
        stride_mb=m.stride(0), stride_mh=m.stride(1), stride_mq=m.stride(2), stride_mk=m.stride(3),
        stride_szb=ks3.stride(0), stride_szh=ks3.stride(1), stride_szn=ks3.stride(2),
        stride_ipb=indptr.stride(0), stride_iph=indptr.stride(1), stride_ipn=indptr.stride(2),
        sm_scale=D ** -0.5, B=1, H=H, S=N, D=D, KC_NUM=cfg.num_k, BLOCK_M=128, BLOCK_N=64)
    out = ref_pm.apply_inverse_permutation_triton(o_fin[None], q_sorted, dim=2)[0]
    lse_orig = torch.empty_like(lse_fin)
    lse_orig.scatter_(1, q_sorted.reshape(H, N).long(), lse_fin)
    store.update(out_rows=f32(out[:, ::8]), lse_rows=lse_orig[:, ::8].numpy(), rows_kept=np.array([8]))
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **store)
    print(f"{name}: {time.time() - t0:.1f}s  map density {m.float().mean():.3f}")


PROC_ROWS_KEPT = 8          # the processor fixtures keep every 8th output row


def _diffusers_stand_ins():
    """The reference's processor modules import a handful of names from diffusers, which is not
    installed here.  None of them is executed on the routes the fixtures take; empty stand-ins let
    the modules import.  `torch.compile` is the identity while they import (they compile
    flex_attention at import time)."""
    import types

    def mod(mname, **attrs):
        m = types.ModuleType(mname)
        m.__dict__.update(attrs)
        sys.modules.setdefault(mname, m)

    att = type("Attention", (torch.nn.Module,), {})
    for name in ("diffusers", "diffusers.models", "diffusers.models.transformers", "diffusers.pipelines",
                 "diffusers.pipelines.hunyuan_video"):
        mod(name)
    mod("diffusers.models.attention_processor", Attention=att)
    mod("diffusers.models.attention", Attention=att)
    mod("diffusers.models.embeddings", apply_rotary_emb=None)
    mod("diffusers.models.normalization", RMSNorm=type("RMSNorm", (torch.nn.Module,), {}))
    mod("diffusers.models.transformers.transformer_wan", _get_added_kv_projections=None, dispatch_attention_fn=None)
    mod("diffusers.pipelines.hunyuan_video.pipeline_hunyuan_video", DEFAULT_PROMPT_TEMPLATE={})


def _import_reference_processors():
    _diffusers_stand_ins()
    real_compile = torch.compile
    torch.compile = lambda f=None, **kw: f
    try:
        import svoo.models.wan.attention as ref_wan
        import svoo.models.hunyuan10.attention as ref_hun
    finally:
        torch.compile = real_compile
    return ref_wan, ref_hun


def _fp32_attention_shim():
    """The Triton interpreter cannot run tl.dot on bf16 operands and the reference's block-sparse
    attention kernel does not up-cast before its dots: it is given the same values as fp32 and
    its result is cast back (the one deviation of layer_case above)."""
    orig = ref_cc.dynamic_block_sparse_fwd_triton

    def shim(q, k, v, *rest, **kw):
        return orig(q.float(), k.float(), v.float(), *rest, **kw).to(q.dtype)

    return shim


def processor_case_wan():
    """The unmodified WanAttn_SAPAttn_Processor.__call__ -> attention_core_logic, configured by
    class attributes the way the installer does it, over four denoising steps of one layer: a
    dense warm-up step, the first clustering, a step that reuses the cached clustering, and a
    re-clustering with kmeans_iter_step iterations; the per-head density comes from a CSV with a
    hole (step 3 falls back to the scalar ratio).  SVG_SPARSE_ATTN_BACKEND=triton selects the
    reference's Triton attention backend (FlashInfer has no CPU path)."""
    from tests import golden_util as gu
    os.environ["SVG_SPARSE_ATTN_BACKEND"] = "triton"
    ref_wan, _ = _import_reference_processors()
    ref_wan.ENABLE_FAST_KERNEL = False                    # norms through the block's own norm modules
    ref_cc.dynamic_block_sparse_fwd_triton = _fp32_attention_shim()
    P = gu.WAN_PROC
    H = P["heads"]
    T, Hh, W = P["grid"]
    N = T * Hh * W
    csv_path = os.path.join(HERE, "processor_wan_density.csv")
    gu.write_density_csv(csv_path, H, [2, 3, 7], hole=(3, 1))
    cls = ref_wan.WanAttn_SAPAttn_Processor
    gu.configure_wan_processor(cls, RefLookup(csv_path))
    cls.measure_attention_sparsity = False
    maps = []
    real_map = ref_wan.identify_dynamic_map

    def recording_map(*a, **kw):
        m = real_map(*a, **kw)
        maps.append((m.clone(), a[5] if len(a) > 5 else kw.get("min_kc_ratio")))
        return m

    ref_wan.identify_dynamic_map = recording_map
    attn = gu.make_attn(31, H)
    cos, sin = gu.rotary_tables(32, N)
    proc = cls(0)
    out = {}
    for i, (step, tval) in enumerate(P["steps"]):
        hidden = gu.wan_step_hidden(step)
        proc._step_from_callback = step
        torch.manual_seed(100 + step)
        n_maps = len(maps)
        t0 = time.time()
        with torch.no_grad():
            y = proc(attn, hidden, rotary_emb=(cos, sin), timestep=torch.tensor([tval]))
        torch.manual_seed(100 + step)                     # the draws co_cluster_tokens made, if it ran
        out[f"q_init_{step}"] = torch.randint(0, N, (H, P["num_q"])).numpy().astype(np.int32)
        out[f"k_init_{step}"] = torch.randint(0, N, (H, P["num_k"])).numpy().astype(np.int32)
        out[f"out_{step}"] = bf16_bits(y[0, ::PROC_ROWS_KEPT])
        out[f"hidden_checksum_{step}"] = checksum(hidden)
        c = getattr(proc, "_cached_clustering_results", None)
        if len(maps) > n_maps:
            m, ratio = maps[-1]
            out[f"map_bits_{step}"] = np.packbits(m.numpy())
            out[f"map_shape_{step}"] = np.array(m.shape)
            out[f"ratio_{step}"] = np.array(ratio if isinstance(ratio, list) else [ratio], dtype=np.float64)
            out[f"qlabels_{step}"] = c["qlabels"].numpy().astype(np.int16)
            out[f"klabels_{step}"] = c["klabels"].numpy().astype(np.int16)
            out[f"qcentroids_{step}"] = bf16_bits(c["qcentroids"])
            out[f"kcentroids_{step}"] = bf16_bits(c["kcentroids"])
            out[f"ksizes_{step}"] = c["kcluster_sizes"].numpy().astype(np.int32)
            out[f"qsizes_{step}"] = c["qcluster_sizes"].numpy().astype(np.int32)
        print(f"processor_wan step {step}: {time.time() - t0:.1f}s, sparse={len(maps) > n_maps}")
    np.savez_compressed(os.path.join(HERE, "processor_wan.npz"), **out)


def processor_case_hunyuan():
    """The unmodified Hunyuan_SAPAttn_Processor2_0.__call__ -> attention_core_logic on a
    single-stream block (text tokens appended after the video tokens), prompt_length <
    context_length so that the unused-prompt block is not empty.  Two substitutions, both needed
    because this route otherwise ends in FlashInfer CUDA code: the module's
    dynamic_block_sparse_fwd_flashinfer name is bound to the reference's own Triton backend
    (same arguments and semantics), and no rotary table is passed (diffusers' apply_rotary_emb
    is not installed)."""
    from tests import golden_util as gu
    _, ref_hun = _import_reference_processors()
    ref_hun.ENABLE_FAST_KERNEL = False
    triton_attn = _fp32_attention_shim()
    ref_hun.dynamic_block_sparse_fwd_flashinfer = lambda q, k, v, m, rs, cs, is_cpu=False: triton_attn(q, k, v, m, rs, cs)
    P = gu.HUN_PROC
    H = P["heads"]
    T, Hh, W = P["grid"]
    N = T * Hh * W
    cls = ref_hun.Hunyuan_SAPAttn_Processor2_0
    gu.configure_hunyuan_processor(cls)
    cls.measure_attention_sparsity = False
    maps = []
    real_map = ref_hun.identify_dynamic_map

    def recording_map(*a, **kw):
        m = real_map(*a, **kw)
        maps.append(m.clone())
        return m

    ref_hun.identify_dynamic_map = recording_map
    attn = gu.make_attn(41, H, joint=True)
    hidden, enc, mask = gu.hunyuan_inputs()
    proc = cls(0)
    step, tval = P["steps"][0]
    proc._step_from_callback = step
    torch.manual_seed(100 + step)
    t0 = time.time()
    with torch.no_grad():
        y, y_enc = proc(attn, hidden, encoder_hidden_states=enc, attention_mask=mask, image_rotary_emb=None,
                        timestep=torch.tensor([tval]))
    torch.manual_seed(100 + step)
    out = dict(q_init=torch.randint(0, N, (H, P["num_q"])).numpy().astype(np.int32),
               k_init=torch.randint(0, N, (H, P["num_k"])).numpy().astype(np.int32))
    c = proc._cached_clustering_results
    m = maps[-1]
    out.update(out=bf16_bits(y[0, ::PROC_ROWS_KEPT]), out_enc=bf16_bits(y_enc[0]), input_checksum=checksum(hidden, enc),
               map_bits=np.packbits(m.numpy()), map_shape=np.array(m.shape),
               qlabels=c["qlabels"].numpy().astype(np.int16), klabels=c["klabels"].numpy().astype(np.int16),
               qcentroids=bf16_bits(c["qcentroids"]), kcentroids=bf16_bits(c["kcentroids"]),
               qsizes=c["qcluster_sizes"].numpy().astype(np.int32), ksizes=c["kcluster_sizes"].numpy().astype(np.int32))
    np.savez_compressed(os.path.join(HERE, "processor_hunyuan.npz"), **out)
    print(f"processor_hunyuan: {time.time() - t0:.1f}s")


def main():
    import dataclasses
    only = sys.argv[1:]
    tiny = synth.LayerConfig("tiny-fp32", 90, 2, (4, 16, 16), torch.float32, 8, 16, 3, (0.25, 0.25), 1, False)
    if only:
        if "euclid" in only:
            euclid_case()
        if "ear" in only:
            from tests import golden_util as gu
            for nm, (cfg, settings) in gu.EAR_CASES.items():
                ear_case(nm, cfg, settings)
        if "processor_wan" in only:
            processor_case_wan()
        if "processor_hunyuan" in only:
            processor_case_hunyuan()
        if "producer" in only:
            producer_case("producer_h6", 96, 6, 21)
            producer_case("producer_h4", 80, 4, 22)
        if "layer_tiny_bf16" in only:
            tiny_b = dataclasses.replace(tiny, name="tiny-bf16", cfg_id=91, dtype=torch.bfloat16, rope=True,
                                         num_q=12, num_k=40, grid=(3, 16, 20))
            layer_case("layer_tiny_bf16", tiny_b, 2, [0.3, 0.15], max_ratio=[0.3, 0.15])
        return
    layer_case("layer_tiny_fp32", tiny, 3, 0.25)
    tiny_b = dataclasses.replace(tiny, name="tiny-bf16", cfg_id=91, dtype=torch.bfloat16, rope=True,
                                 num_q=12, num_k=40, grid=(3, 16, 20))
    layer_case("layer_tiny_bf16", tiny_b, 2, [0.3, 0.15], max_ratio=[0.3, 0.15])
    layer_case("layer_cfg0", synth.CONFIGS["cfg0"], 10, 0.20, rows_kept=32, max_ratio=0.20)
    map_case("map_bf16_budget", 4, 100, 500, torch.bfloat16, 0.9, [0.07, 0.12, 0.2, 0.25], [0.07, 0.12, 0.2, 0.25], 11)
    map_case("map_bf16_topp_floor", 4, 100, 500, torch.bfloat16, 0.9, [0.15, 0.2, 0.0, 0.18], None, 12)
    map_case("map_bf16_scalar", 3, 64, 256, torch.bfloat16, 0.88, 0.1, None, 13)
    map_case("map_fp32_topp", 2, 32, 128, torch.float32, 0.9, 0, None, 14)
    map_case("map_fp32_cap_scalar", 2, 32, 128, torch.float32, 0.95, [0.1, 0.3], 0.2, 15)
    map_case("map_bf16_big", 2, 256, 1024, torch.bfloat16, 0.9, [0.15, 0.2], None, 16)
    map_case("map_all_ones", 2, 8, 16, torch.bfloat16, 1.0, 0.1, None, 17)
    lookup_case()
    producer_case("producer_h6", 96, 6, 21)
    producer_case("producer_h4", 80, 4, 22)


if __name__ == "__main__":
    main()
