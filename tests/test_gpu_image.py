"""Layer images on the GPU: every matrix of an image arrives in HBM bit-exact
(whole and as the row slice a rank owns), and the image checks itself the way the
reference's packer intends: fused gate/up on the packer's sin/cos activation
reproduces the eight reference rows stored in the header
(qwen38_m3_pack.c:187-239, header field source_reference_first_8)."""
import importlib

import numpy as np
import pytest

from q4_cases import assert_close, bits_equal

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx(q4b):
    context = q4b.Q4Context(0)
    yield context
    context.close()


@pytest.fixture(scope="module")
def image(q4b):
    return importlib.import_module("cpu-llms-in-c_b200.image")


def build(orc, image, path, kind, layer, hidden, intermediate, input_rows, output_groups, seed):
    shapes = [(intermediate, hidden // 64), (intermediate, hidden // 64), (hidden, intermediate // 64),
              (input_rows, hidden // 64), (hidden, output_groups)]
    matrices = {m: orc.synth_weight(seed, m, rows, groups) for m, (rows, groups) in enumerate(shapes)}
    x = orc.activation_sincos(hidden).reshape(1, hidden)
    (gq, gm), (uq, um) = matrices[image.GATE], matrices[image.UP]
    reference, _ = orc.gate_up_silu(gq[:8], gm[:8], uq[:8], um[:8], hidden // 64, x, want64=False)
    image.write_layer_image(path, kind, layer, hidden, intermediate, matrices,
                            np.linspace(0, 1, 64, dtype=np.float32), gate_up_reference=reference[0])
    return matrices, x


@pytest.mark.parametrize("kind_name,layer", [("DELTA", 2), ("ATTENTION", 3)])
def test_image_matrices_arrive_bit_exact(q4b, orc, ctx, image, tmp_path, kind_name, layer):
    kind = getattr(image, kind_name)
    path = str(tmp_path / "layer.img")
    matrices, _ = build(orc, image, path, kind, layer, 1024, 3072, 2112, 32, seed=layer)
    opened = image.Q4Image(path, kind, layer)
    for m, (quants, meta) in matrices.items():
        rows, groups = opened.shape(m)
        weight = opened.weight(ctx, m)
        codes, w32, w16 = weight.unpack()
        assert (codes == orc.unpack_codes(quants, rows, groups)).all()
        assert bits_equal(w32, orc.dequant_w32(quants, meta, rows, groups))
        assert bits_equal(w16, orc.dequant_w16(quants, meta, rows, groups))
        weight.free()
        # the slice of the second of three ranks
        begin, count = (rows // 48) * 16, (rows // 48) * 16
        part = opened.weight(ctx, m, begin, count)
        _, w32, _ = part.unpack(codes=False, w16=False)
        assert bits_equal(w32, orc.dequant_w32(quants, meta, rows, groups)[begin:begin + count])
        part.free()
    opened.close()


def test_image_reproduces_its_embedded_reference(q4b, orc, ctx, image, tmp_path):
    path = str(tmp_path / "layer.img")
    hidden, intermediate = 5120, 1024  # the packer's hidden size; a short intermediate keeps the file small
    matrices, x = build(orc, image, path, image.DELTA, 0, hidden, intermediate, 256, 4, seed=9)
    opened = image.Q4Image(path, image.DELTA, 0)
    assert list(opened.info.reference_counts)[:1] == [8]
    gate, up = opened.weight(ctx, image.GATE), opened.weight(ctx, image.UP)
    dx = ctx.to_device(x)
    dy = ctx.alloc(intermediate * 4)
    ctx.gate_up_silu(gate, up, dx.ptr, q4b.F16, 1, dy.ptr, q4b.F32)
    got = dy.download(np.float32, (1, intermediate))
    stored = np.array(list(opened.info.gate_up_reference_first_8), dtype=np.float32).reshape(1, 8)
    assert_close(got[:, :8], stored, "first eight rows against the header's reference")
    # and the down projection of the same image against the oracle
    (dq, dm) = matrices[image.DOWN]
    down = opened.weight(ctx, image.DOWN)
    h = orc.synth_x(9, 0, 4, intermediate)
    dh = ctx.to_device(h)
    dz = ctx.alloc(4 * hidden * 2)
    ctx.matmul(down, dh.ptr, q4b.F16, 4, dz.ptr, q4b.F16)
    _, want = orc.matmul(dq, dm, intermediate // 64, h, want32=False)
    assert_close(dz.download(np.float16, (4, hidden)), want, "down projection from the image")
    for weight in (gate, up, down):
        weight.free()
    opened.close()


def oracle_mlp(orc, matrices, image, hidden, intermediate, x, residual):
    """silu(gate x) * (up x) in fp32, then down on that fp32 vector plus residual, as the
    reference's decode MLP does (qwen38_q4_gate_up_silu, qwen38_q4_mlp_down_residual_f32)."""
    (gq, gm), (uq, um), (dq, dm) = matrices[image.GATE], matrices[image.UP], matrices[image.DOWN]
    mid32, _ = orc.gate_up_silu(gq, gm, uq, um, hidden // 64, x, want64=False)
    _, out = orc.matmul(dq, dm, intermediate // 64, mid32, residual=residual, want32=False)
    return mid32, out


@pytest.mark.parametrize("batch", [1, 4, 40])
def test_layer_encoders_from_an_image(q4b, orc, ctx, image, tmp_path, batch):
    hidden, intermediate, input_rows, output_groups = 1024, 3072, 2112, 32
    path = str(tmp_path / "layer.img")
    matrices, _ = build(orc, image, path, image.DELTA, 4, hidden, intermediate, input_rows, output_groups, seed=4)
    opened = image.Q4Image(path, image.DELTA, 4)
    x = orc.synth_x(4, 0, batch, hidden)
    residual = orc.synth_x(4, 7, batch, hidden).astype(np.float32)
    mixer = orc.synth_x(4, 8, batch, output_groups * 64).astype(np.float32)
    mid_ref, out_ref = oracle_mlp(orc, matrices, image, hidden, intermediate, x, residual)
    _, in_ref = orc.matmul(*matrices[image.INPUT], hidden // 64, x, want32=False)
    _, o_ref = orc.matmul(*matrices[image.OUTPUT], output_groups, mixer, residual=residual, want32=False)

    dx, dres, dmix = ctx.to_device(x), ctx.to_device(residual), ctx.to_device(mixer)
    for world in (1, 2, 3):
        dmid = ctx.to_device(np.zeros((batch, intermediate), np.float32))
        dout = ctx.to_device(np.zeros((batch, hidden), np.float32))
        din = ctx.to_device(np.zeros((batch, input_rows), np.float16))
        dhid = ctx.to_device(np.zeros((batch, hidden), np.float32))
        layers = [image.Q4LayerMatmuls.load(ctx, opened, rank, world) for rank in range(world)]
        if world == 1:
            layers[0].encode_mlp(dx.ptr, batch, dmid.ptr, q4b.F32, dres.ptr, q4b.F32, dout.ptr, q4b.F32)
        else:
            with pytest.raises(q4b.Q4Error):
                layers[0].encode_mlp(dx.ptr, batch, dmid.ptr, q4b.F32, dres.ptr, q4b.F32, dout.ptr, q4b.F32)
            for layer in layers:      # every rank's slice of the intermediate lands in the same buffer: the gather
                layer.encode_gate_up(dx.ptr, batch, dmid.ptr, q4b.F32)
            for layer in layers:
                layer.encode_down(dmid.ptr, q4b.F32, batch, dres.ptr, q4b.F32, dout.ptr, q4b.F32)
        for layer in layers:
            layer.encode_input(dx.ptr, batch, din.ptr, q4b.F16)
            layer.encode_output(dmix.ptr, q4b.F32, batch, dres.ptr, q4b.F32, dhid.ptr, q4b.F32)
        assert_close(dmid.download(np.float32, (batch, intermediate)), mid_ref.astype(np.float64), f"gate/up world {world}")
        assert_close(dout.download(np.float32, (batch, hidden)), out_ref, f"mlp world {world}")
        assert_close(din.download(np.float16, (batch, input_rows)), in_ref, f"in-projection world {world}")
        assert_close(dhid.download(np.float32, (batch, hidden)), o_ref, f"out-projection world {world}")
        for layer in layers:
            layer.free()
    opened.close()


def test_embedding_lookup_from_a_global_image(q4b, orc, ctx, image, tmp_path):
    vocab, hidden = 3001, 1024
    embedding = orc.synth_weight(6, 0, vocab, hidden // 64)
    lm_head = orc.synth_weight(6, 1, vocab, hidden // 64)
    path = str(tmp_path / "global.img")
    image.write_global_image(path, hidden, embedding, lm_head, np.ones(hidden, np.float32))
    opened = image.Q4Image(path, image.GLOBAL, 0)
    tokens = np.array([0, 1, 15, 16, 17, 2999, 3000, 1234, 1234, 64, 127, 128], dtype=np.uint32)
    w32 = orc.dequant_w32(*embedding, vocab, hidden // 64)
    d_tokens = ctx.to_device(tokens)
    whole = opened.weight(ctx, image.EMBEDDING)
    out16, out32 = ctx.alloc(tokens.size * hidden * 2), ctx.alloc(tokens.size * hidden * 4)
    ctx.embedding_lookup(whole, d_tokens.ptr, tokens.size, out32.ptr, q4b.F32)
    ctx.embedding_lookup(whole, d_tokens.ptr, tokens.size, out16.ptr, q4b.F16)
    assert bits_equal(out32.download(np.float32, (tokens.size, hidden)), w32[tokens])
    assert bits_equal(out16.download(np.float16, (tokens.size, hidden)), w32[tokens].astype(np.float16))
    # a vocabulary split over three ranks: every shard answers for its rows and writes zeros elsewhere
    total = np.zeros((tokens.size, hidden), dtype=np.float32)
    for rank in range(3):
        begin, count = image.Q4LayerMatmuls.slice_of(vocab, rank, 3)
        shard = opened.weight(ctx, image.EMBEDDING, begin, count)
        ctx.embedding_lookup(shard, d_tokens.ptr, tokens.size, out32.ptr, q4b.F32)
        total += out32.download(np.float32, (tokens.size, hidden))
        shard.free()
    assert bits_equal(total, w32[tokens])
    # and the lm_head of the same image as a matmul
    head = opened.weight(ctx, image.LM_HEAD)
    x = orc.synth_x(6, 0, 1, hidden)
    dx, dy = ctx.to_device(x), ctx.alloc(vocab * 4)
    ctx.matmul(head, dx.ptr, q4b.F16, 1, dy.ptr, q4b.F32)
    _, want = orc.matmul(*lm_head, hidden // 64, x, want32=False)
    assert_close(dy.download(np.float32, (1, vocab)), want, "lm_head from the global image")
    for weight in (whole, head):
        weight.free()
    opened.close()


@pytest.mark.parametrize("batch", [1, 4, 40])
def test_fc_projection_from_an_mtp_extras_image(q4b, orc, ctx, image, tmp_path, batch):
    """encode_mtp_pass feeds concat[embedding norm, hidden norm] (2 x hidden) through the fc matrix
    (qwen38_m3_decode.m:1818-1821); here by row slice over two ranks as well."""
    hidden = 1024
    fc = orc.synth_weight(13, 0, hidden, 2 * hidden // 64)
    path = str(tmp_path / "mtp.img")
    image.write_mtp_image(path, hidden, fc, *[np.ones(hidden, np.float32)] * 3)
    opened = image.Q4Image(path, image.MTP, 0)
    x = orc.synth_x(13, batch, batch, 2 * hidden)
    _, want = orc.matmul(*fc, 2 * hidden // 64, x, want32=False)
    dx = ctx.to_device(x)
    whole = opened.weight(ctx, image.FC)
    dy = ctx.alloc(batch * hidden * 4)
    ctx.matmul(whole, dx.ptr, q4b.F16, batch, dy.ptr, q4b.F32)
    assert_close(dy.download(np.float32, (batch, hidden)), want, "fc from the MTP extras image")
    whole.free()
    if batch <= 16:
        for rank in range(2):
            begin, count = image.Q4LayerMatmuls.slice_of(hidden, rank, 2)
            shard = opened.weight(ctx, image.FC, begin, count)
            part = ctx.alloc(batch * count * 4)
            ctx.matmul(shard, dx.ptr, q4b.F16, batch, part.ptr, q4b.F32)
            assert_close(part.download(np.float32, (batch, count)), want[:, begin:begin + count], f"fc rows of rank {rank}")
            shard.free()
    opened.close()
