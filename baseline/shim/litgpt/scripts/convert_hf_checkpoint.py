"""Stand-in for ``litgpt.scripts.convert_hf_checkpoint``."""
import torch


def qkv_reassemble(param: torch.Tensor, config) -> torch.Tensor:
    """Turns a per-group interleaved ``[q…q k v]`` QKV weight (or bias) into the ``[Q | K | V]`` layout."""
    q_per_kv = config.n_head // config.n_query_groups
    qs, ks, vs = [], [], []
    for chunk in torch.chunk(param, config.n_query_groups):
        q, k, v = torch.split(chunk, [config.head_size * q_per_kv, config.head_size, config.head_size])
        qs.append(q)
        ks.append(k)
        vs.append(v)
    return torch.cat((torch.cat(qs), torch.cat(ks), torch.cat(vs)))
