"""The operator set DiTStack needs, served by the CPU oracle (test infrastructure only).

Same names and argument meaning as comfy_kitchen.backends.cuda, so the stack's host logic
(sharding, scales, collectives) can run on CPU ranks."""
import torch
import torch.nn.functional as F

from oracle import ck_oracle as orc


def quantize_nvfp4(x, per_tensor_scale, epsilon=0.0, pad_16x=False, hi_first=True):
    return orc.quantize_nvfp4(x, per_tensor_scale, epsilon, pad_16x, hi_first)


def dequantize_nvfp4(qx, per_tensor_scale, block_scales, output_type=torch.bfloat16, hi_first=True):
    return orc.dequantize_nvfp4(qx, per_tensor_scale, block_scales, output_type, hi_first)


def scaled_mm_nvfp4(a, b, tensor_scale_a, tensor_scale_b, block_scale_a, block_scale_b, bias=None,
                    out_dtype=torch.bfloat16, alpha=None, out=None):
    y = orc.scaled_mm_nvfp4(a, b, tensor_scale_a, tensor_scale_b, block_scale_a, block_scale_b,
                            bias=bias, out_dtype=out_dtype, alpha=alpha)
    if out is not None:
        out.copy_(y)
        return out
    return y


def adaln(x, scale, shift, eps=1e-6):
    return orc.adaln(x, scale, shift, eps, single_rounding=True)


def adaln_quantize_nvfp4(x, scale, shift, per_tensor_scale, eps=1e-6, hi_first=True):
    y = adaln(x, scale, shift, eps)
    return orc.quantize_nvfp4(y.reshape(-1, y.shape[-1]), per_tensor_scale, 0.0, False, hi_first)


def rmsnorm(x, weight=None, eps=1e-6):
    w = None if weight is None else weight.float()
    return F.rms_norm(x.float(), (x.shape[-1],), w, eps).to(x.dtype)


def apply_rope(xq, xk, freqs_cis):
    return orc.apply_rope(xq.contiguous(), xk.contiguous(), freqs_cis.contiguous())


def qk_norm_rope(qkv, q_weight, k_weight, freqs_cis, heads, q_out=None, k_out=None, v_out=None, token_offset=0,
                 eps=1e-6):
    """rms_norm (fp32, one rounding) of q and k per head, then the oracle's rope, then the attention layout."""
    t, total = qkv.shape[0], freqs_cis.shape[2]
    q, k, v = qkv[:, :3 * heads * 128].reshape(t, 3, heads, 128).unbind(1)
    q = rmsnorm(q, q_weight, eps).permute(1, 0, 2)[None].contiguous()
    k = rmsnorm(k, k_weight, eps).permute(1, 0, 2)[None].contiguous()
    f = freqs_cis[:, :, token_offset:token_offset + t].contiguous()
    q, k = orc.apply_rope(q, k, f)
    outs = []
    for o, val in ((q_out, q), (k_out, k), (v_out, v.permute(1, 0, 2)[None])):
        if o is None:
            o = torch.zeros((1, heads, total, 128), dtype=qkv.dtype)
        o[:, :, token_offset:token_offset + t] = val
        outs.append(o)
    return tuple(outs)


def _gathered(segments):
    cols = []
    for t, act in segments:
        m = t if t.dim() == 2 else t.permute(1, 0, 2).reshape(t.shape[1], -1)
        if act == "gelu_tanh":
            m = F.gelu(m.float(), approximate="tanh").to(t.dtype)
        cols.append(m)
    return torch.cat(cols, dim=1).contiguous()


def quantize_nvfp4_gather(segments, per_tensor_scale, hi_first=True):
    return orc.quantize_nvfp4(_gathered(segments), per_tensor_scale, 0.0, False, hi_first)
