"""FLOP accounting of the reference (kvax/utils/math.py:1-30)."""


def get_multi_head_attention_tflops(batch_size, query_seq_len, kv_seq_len, num_heads, qk_head_dim,
                                    value_head_dim, causal, num_gpus=1, forward_pass=True, backward_pass=False):
    if not forward_pass and not backward_pass:
        raise ValueError("At least one of the forward_pass or backward_pass should be True")
    result = batch_size * num_heads * 2 * (qk_head_dim + value_head_dim) * query_seq_len * kv_seq_len / 1e12
    if causal:
        result *= 0.5
    if forward_pass and backward_pass:
        result *= 3.5
    elif backward_pass:
        result *= 2.5
    return result / num_gpus
