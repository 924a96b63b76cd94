"""Writes oracle/_ref/modern_gpt_engine.cu: the reference's ModernGPT (llm/src/model/modern_gpt.cu, read from the
reference tree where it lies, never stored in this repository) with its attention chain replaced by calls into
modern-llm-v1_b200/csrc/modernllm_chain.h.  Only the REPLACEMENT text lives here; the ranges that go are named by
line number and checked against identifiers the reference has on their first and last lines, so another revision
of the reference fails loudly instead of being patched wrongly.

    python oracle/model_patch.py <reference llm dir> <output .cu> [--bf16-io]

--bf16-io additionally switches the q/k/v/o projections to the reference's BF16-in/BF16-out linear layers
(linear_forward_bf16inout / linear_backward_bf16inout, llm/src/model/linear.h:71-83) so that no FP32<->BF16 cast is
left around attention.
"""
import sys

TINY = "{1}"

# (first line, last line, text that must occur on the first line, on the last line, replacement)
def edits(bf16_io: bool):
    fwd_call = (
        "    b200::chain_attention_forward(this, {q}, {k}, {v}, rope_cos_, rope_sin_, bl.q_norm_g, bl.k_norm_g, 1e-5f,\n"
        "                                  bl.q_norm_rstd, bl.k_norm_rstd, {ctx}, B, T, H, n_kv_, d_h_);\n")
    bwd_call = (
        "        b200::chain_attention_backward(this, {d_ctx}, {q}, {k}, {v}, {ctx}, rope_cos_, rope_sin_, bl.q_norm_g,\n"
        "                                       bl.k_norm_g, bl.q_norm_rstd, bl.k_norm_rstd, {dq}, {dk}, {dv},\n"
        "                                       bl.d_q_norm_g, bl.d_k_norm_g, B, T, H, n_kv_, d_h_);\n")
    if not bf16_io:
        fwd = fwd_call.format(q="bl.q_proj", k="bl.k_proj", v="bl.v_proj", ctx="bl.ctx")
        bwd = bwd_call.format(d_ctx="d_ctx_", q="bl.q_proj", k="bl.k_proj", v="bl.v_proj", ctx="bl.ctx", dq="d_q_proj_",
                              dk="d_k_proj_", dv="d_v_proj_")
        out = [
            (351, 378, "Tensor q3 = bl.q_proj.view", "merge_heads(bl.ctx_split, bl.ctx", fwd),
            (505, 552, "Tensor d_ctx_split(", "merge_heads(d_v_split_, dvp3", bwd),
        ]
    else:
        # BF16 projections: X (ln1_out) is cast once, the three projections and the output projection run BF16 in / BF16
        # out, and the chain passes their buffers straight to the engine.
        fwd = (
            "    b200::ChainIo& io = b200::chain_io(this, B * T, D, Dkv);\n"
            "    cast_fp32_to_bf16(bl.ln1_out, io.x);\n"
            "    linear_forward_bf16inout(handle, io.x, bl.Wq_bf16, nullptr, io.q_proj);\n"
            "    linear_forward_bf16inout(handle, io.x, bl.Wk_bf16, nullptr, io.k_proj);\n"
            "    linear_forward_bf16inout(handle, io.x, bl.Wv_bf16, nullptr, io.v_proj);\n"
            + fwd_call.format(q="io.q_proj", k="io.k_proj", v="io.v_proj", ctx="io.ctx") +
            "    linear_forward_bf16inout(handle, io.ctx, bl.Wo_bf16, nullptr, io.attn_out);\n"
            "    cast_bf16_to_fp32(io.attn_out, bl.attn_out);\n")
        bwd = (
            "        b200::ChainIo& io = b200::chain_io(this, B * T, D, n_kv_ * d_h_);\n"
            "        cast_fp32_to_bf16(d_attn_out_, io.d_attn_out);\n"
            "        linear_backward_bf16inout(handle, io.ctx, bl.Wo_bf16, io.d_attn_out, io.d_ctx, bl.d_Wo, nullptr);\n"
            + bwd_call.format(d_ctx="io.d_ctx", q="io.q_proj", k="io.k_proj", v="io.v_proj", ctx="io.ctx", dq="io.d_q_proj",
                              dk="io.d_k_proj", dv="io.d_v_proj") +
            "        linear_backward_bf16inout(handle, io.x, bl.Wq_bf16, io.d_q_proj, io.d_x, bl.d_Wq, nullptr);\n"
            "        cast_bf16_to_fp32(io.d_x, d_ln1_out_);\n"
            "        linear_backward_bf16inout(handle, io.x, bl.Wk_bf16, io.d_k_proj, io.d_x, bl.d_Wk, nullptr);\n"
            "        cast_bf16_to_fp32(io.d_x, d_branch_);\n"
            "        add_inplace(d_ln1_out_, d_branch_);\n"
            "        linear_backward_bf16inout(handle, io.x, bl.Wv_bf16, io.d_v_proj, io.d_x, bl.d_Wv, nullptr);\n"
            "        cast_bf16_to_fp32(io.d_x, d_branch_);\n"
            "        add_inplace(d_ln1_out_, d_branch_);\n")
        out = [
            # the three projections, the head split ... merge, and the output projection
            (347, 380, "lin_fwd(bl.ln1_out, bl.Wq", "lin_fwd(ctx_flat, bl.Wo", fwd),
            # the output projection's backward ... the three projections' backward
            (501, 561, "Tensor d_ctx_flat = d_ctx_.view", "add_inplace(d_ln1_out_, d_branch_);", bwd),
        ]
    # buffers of the replaced chain that the model no longer needs (they stay declared; one element each)
    for first, last, a, b in ((74, 78, "alloc(d_q_split_", "alloc(d_v_split_"), (94, 98, "alloc(act_q_split_", "alloc(act_k_normed_"),
                              (101, 104, "alloc(act_k_full_", "alloc(act_probs_")):
        out.append((first, last, a, b, None))
    return out


def main():
    ref, dst = sys.argv[1], sys.argv[2]
    bf16_io = "--bf16-io" in sys.argv[3:]
    path = f"{ref}/src/model/modern_gpt.cu"
    lines = open(path).read().split("\n")
    plan = sorted(edits(bf16_io), key=lambda e: -e[0])  # bottom up, so that line numbers stay valid
    for first, last, a, b, text in plan:
        if a not in lines[first - 1] or b not in lines[last - 1]:
            raise SystemExit(f"{path}: lines {first}-{last} are not what this patch expects "
                             f"({a!r} ... {b!r}); a different revision of the reference?")
        if text is None:  # allocation lines: keep the tensor, shrink it to one element
            new = []
            for ln in lines[first - 1:last]:
                name = ln.split("alloc(")[1].split(",")[0]
                new.append(f"    alloc({name}, {TINY});")
        else:
            new = text.rstrip("\n").split("\n")
        lines[first - 1:last] = new
    # the chain's header, after the reference's own includes
    at = max(i for i, ln in enumerate(lines) if ln.startswith("#include"))
    lines.insert(at + 1, '#include "modernllm_chain.h"')
    with open(dst, "w") as f:
        f.write("// GENERATED by oracle/model_patch.py from the reference's llm/src/model/modern_gpt.cu; not stored in git.\n")
        f.write("\n".join(lines))


if __name__ == "__main__":
    main()
