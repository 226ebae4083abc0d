"""The arrangement of a layer's branches, on the CPU with stand-in parts."""
import torch


def test_residual_arrangement_fuses_the_addition_with_the_next_norm():
    """Two branches behind a norm each (the reference's block): h += pending; a =
    mixer(norm(h)); h += a; returns ffn(norm(h)) unadded.  Then a branch without a norm and
    one with a norm after the part."""
    from cretif_b200.engine.model import Branch, Layer
    from cretif_b200.parts.base import lookup_part

    class Norm:
        def forward(self, h, delta=None, rows=None, write_h=True):
            if delta is not None:
                h += delta
            return h * 2

    class Mixer:
        dtype = torch.float32

        def forward(self, x, ctx, cache):
            return x + 1

    class FF:
        dtype = torch.float32

        def forward(self, x, ctx):
            return x * 10

    run = lookup_part("arrangement", "residual")
    layer = Layer("", [Branch("mixer", Mixer(), Norm()), Branch("feed_forward", FF(), Norm())], run)
    h = torch.ones(2, 3)
    out = run(layer, h, torch.full((2, 3), 0.5), None, [None, None])
    # h = 1.5; a = 2*1.5 + 1 = 4; h = 5.5; out = 10 * (2 * 5.5) = 110
    assert torch.allclose(h, torch.full((2, 3), 5.5)) and torch.allclose(out, torch.full((2, 3), 110.0))
    # one branch, no norm before it, a norm after it: out = 2 * (h + 1) with h = 1 + 0.5
    layer = Layer("", [Branch("mixer", Mixer(), None, Norm())], run)
    h = torch.ones(2, 3)
    out = run(layer, h, torch.full((2, 3), 0.5), None, [None])
    assert torch.allclose(h, torch.full((2, 3), 1.5)) and torch.allclose(out, torch.full((2, 3), 5.0))
