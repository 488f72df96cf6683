"""The way of the weights to the device (GPU): through pinned buffers in chunks, bit for bit what a plain copy gives."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_uploader_copies_every_size_and_type_bit_for_bit():
    from lucciola_b200.weights.loader import Uploader
    dev = torch.device("cuda:0")
    up = Uploader(dev, threads=3)
    up.CHUNK = 1 << 20                      # small chunks: several per tensor, sizes that are no multiple of a chunk or a thread's share
    up._pinned = [torch.empty(up.CHUNK, dtype=torch.uint8, pin_memory=True) for _ in range(2)]
    g = torch.Generator().manual_seed(0)
    cases = [((7,), torch.float32), ((1 << 19,), torch.bfloat16), ((1025, 1027), torch.bfloat16), ((3, 1 << 20), torch.float16),
             ((2_500_001,), torch.float32), ((1 << 21, 3), torch.int32), ((1 << 22,), torch.uint8)]
    for shape, dtype in cases:
        if dtype.is_floating_point:
            t = torch.randn(shape, generator=g).to(dtype)
        else:
            t = torch.randint(0, 100, shape, generator=g).to(dtype)
        got = up.upload(t)
        torch.cuda.synchronize()
        assert got.dtype == dtype and got.shape == t.shape and got.device.type == "cuda"
        assert torch.equal(got.cpu().view(torch.uint8), t.view(torch.uint8)), (shape, dtype)
    # a view that is not contiguous goes the plain way
    t = torch.randn(2048, 2048, generator=g).t()
    assert torch.equal(up.upload(t).cpu(), t)
    up.close()


def test_a_model_folder_loads_through_the_uploader(tmp_path):
    """Tensors larger than a chunk, fused and plain, in both engine types: the parts hold what the files hold."""
    from lucciola_b200.config import EngineOptions
    from lucciola_b200.engine.load import build_runner
    from lucciola_b200.weights import CheckpointFolder, write_random_model
    from lucciola_b200.weights import loader
    cfg = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 1, "hidden_size": 1024,
           "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 3072, "vocab_size": 5000,
           "rope_theta": 1e6, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 256,
           "hidden_act": "silu", "attention_bias": False}
    write_random_model(cfg, tmp_path, 3, std=0.02, norm_std=0.05)
    old = loader.Uploader.CHUNK
    loader.Uploader.CHUNK = 1 << 20
    try:
        src = CheckpointFolder(tmp_path)
        for dtype in ("bfloat16", "float32"):
            r = build_runner(tmp_path, EngineOptions(dtype=dtype, max_blocks=8))
            want = src.get("model.embed_tokens.weight")
            got = r.model.embedding.weight
            assert torch.equal(got.cpu().float(), want.float())
            o = r.model.blocks[0].mixer.o.weight
            assert torch.equal(o.cpu().float(), src.get("model.layers.0.self_attn.o_proj.weight").float())
    finally:
        loader.Uploader.CHUNK = old
