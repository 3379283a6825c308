"""Train a small text-conditioned flow-matching DiT on synthetic captioned images, then serve prompts through the
text-to-image task (classifier-free guidance, per-request settings) and write a PNG grid.  Counterpart of the reference's
examples/sample_text_to_image.py.

    python examples/sample_text_to_image.py [--steps 300] [--device cuda] [--out grid.png]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import dew_b200 as dew
from dew_b200.diffusion import presets
from dew_b200.inference.images import ImageRequest, ImageSettings, TextToImage, serve
from dew_b200.inputs import Condition, Field, InputSpec
from dew_b200.models.dit import SimpleDiT
from dew_b200.objectives.diffusion import DiffusionObjective
from dew_b200.sampling import CFG, Euler

COLOURS = {"red": (0.9, -0.8, -0.8), "green": (-0.8, 0.9, -0.8), "blue": (-0.8, -0.8, 0.9)}
SHAPES = ("square", "stripe")


class Words:
    """Caption -> bag-of-words features over the tiny vocabulary (a stand-in for a text encoder)."""
    vocab = list(COLOURS) + list(SHAPES)

    def __call__(self, captions):
        out = torch.zeros(len(captions), len(self.vocab))
        for i, c in enumerate(captions):
            for j, w in enumerate(self.vocab):
                out[i, j] = float(w in c)
        return out


def dataset(n, g):
    images, captions = torch.full((n, 16, 16, 3), -0.9), []
    for i in range(n):
        colour = list(COLOURS)[int(torch.randint(0, 3, (), generator=g))]
        shape = SHAPES[int(torch.randint(0, 2, (), generator=g))]
        rgb = torch.tensor(COLOURS[colour])
        if shape == "square":
            images[i, 4:12, 4:12] = rgb
        else:
            images[i, :, 6:10] = rgb
        captions.append(f"a {colour} {shape}")
    return images, captions


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--out", default=None)
    args = ap.parse_args(argv)
    dev = torch.device(args.device)
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(0)
    words = Words()
    model = SimpleDiT(patch_size=4, emb_features=64, num_layers=3, num_heads=2, text_features=len(words.vocab)).to(dev)
    inputs = InputSpec(Field("sample", (16, 16, 3)), {"text": Condition(Field("text", ()), encoder=lambda c: words(c).to(dev) if not torch.is_tensor(c) else c)})
    objective = DiffusionObjective(model, presets.Flow(), inputs, ema_decay=None, solver=Euler(), guidance=CFG(2.0), steps=12,
                                   unconditional_prob=0.15)
    images, captions = dataset(512, g)
    feats = words(captions)
    data = [{"sample": images[i:i + 32].to(dev), "text": feats[i:i + 32].to(dev)} for i in range(0, 512, 32)]
    trainer = dew.Trainer(objective, dew.OptimConfig(learning_rate=2e-3), key=0, tracker=dew.MemoryTracker())
    trainer.fit(data * (args.steps // len(data) + 1), steps=args.steps, log_every=max(1, args.steps // 5))
    task = TextToImage.from_objective(objective)
    prompts = [f"a {c} {s}" for c in COLOURS for s in SHAPES]
    answers = serve(task, [ImageRequest(prompts, key=1), ImageRequest(prompts[:2], key=2, settings=ImageSettings(steps=6, guidance=None))])
    out = answers[0].decoded.cpu()
    # how often the brightest channel of the painted region is the prompted colour
    hits = 0
    for img, p in zip(out, prompts):
        region = img[6:10, 6:10].mean((0, 1))
        hits += int(list(COLOURS)[int(region.argmax())] in p)
    if args.out:
        from dew_b200.utils.artifacts import ImageGrid
        ImageGrid(out).save(args.out)
    print(f"{hits} of {len(prompts)} prompts drew their colour; unguided 6-step request: {tuple(answers[1].decoded.shape)}")
    return hits, len(prompts)


if __name__ == "__main__":
    main()
