"""Parameter shape lists of the GPT-style models the benchmark configurations
name, in Hugging Face GPT-2 module order, for building chunk layouts without
instantiating a model.  Group 0 = tensors with weight decay (>= 2-D weights),
group 1 = biases and LayerNorm parameters (no decay).  The reference's own
model table lives in examples/model_builder.py:36-202 (hidden size, layer
count, sequence length per named model)."""


def gpt_tensor_specs(n_layer, hidden, vocab=50257, n_pos=1024):
    """List of (name, shape, group) in module order: wte, wpe, the blocks, ln_f."""
    h = hidden
    specs = [("wte.weight", (vocab, h), 0), ("wpe.weight", (n_pos, h), 0)]
    for i in range(n_layer):
        p = "h.%d." % i
        specs += [
            (p + "ln_1.weight", (h,), 1), (p + "ln_1.bias", (h,), 1),
            (p + "attn.c_attn.weight", (h, 3 * h), 0), (p + "attn.c_attn.bias", (3 * h,), 1),
            (p + "attn.c_proj.weight", (h, h), 0), (p + "attn.c_proj.bias", (h,), 1),
            (p + "ln_2.weight", (h,), 1), (p + "ln_2.bias", (h,), 1),
            (p + "mlp.c_fc.weight", (h, 4 * h), 0), (p + "mlp.c_fc.bias", (4 * h,), 1),
            (p + "mlp.c_proj.weight", (4 * h, h), 0), (p + "mlp.c_proj.bias", (h,), 1),
        ]
    specs += [("ln_f.weight", (h,), 1), ("ln_f.bias", (h,), 1)]
    return specs


MODELS = {
    # name: (n_layer, hidden, vocab, n_pos)
    "gpt2_1.5b": (48, 1600, 50257, 1024),
    "gpt_12b": (40, 5120, 50257, 1024),
    "gpt_40b": (48, 8192, 50257, 1024),
}


def model_specs(name):
    n_layer, hidden, vocab, n_pos = MODELS[name]
    return gpt_tensor_specs(n_layer, hidden, vocab, n_pos)
