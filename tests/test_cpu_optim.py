

def test_flat_buffer_takes_the_weights_dtype_not_the_first_parameters():
    """A small fp32 parameter that sorts first (tensor-parallel replicated class) must not turn the whole buffer - and with it
    every weight - into fp32."""
    import torch
    from elfa_b200.optim.flat import FlatParams
    beta = torch.nn.Parameter(torch.ones(1, dtype=torch.float32))
    beta.tp_replicated = True
    beta.no_decay = True
    w1 = torch.nn.Parameter(torch.randn(64, 32).to(torch.bfloat16))
    w2 = torch.nn.Parameter(torch.randn(32, 64).to(torch.bfloat16))
    flat = FlatParams([("w1", w1), ("beta", beta), ("w2", w2)])
    assert flat.names[0] == "beta"                       # the replicated class leads the order
    assert flat.dtype == torch.bfloat16 and flat.flat.dtype == torch.bfloat16
    assert w1.dtype == torch.bfloat16 and w2.dtype == torch.bfloat16 and beta.dtype == torch.bfloat16
    assert float(beta.detach()) == 1.0
