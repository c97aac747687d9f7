"""Vision tower pieces on CPU: preprocessing, tower shapes and invariances, scatter, m-RoPE ids, cache."""
import numpy as np
import pytest
import torch

from owl_engine_b200.cli import png
from owl_engine_b200.models import vision as V


def test_smart_resize_bounds():
    assert V.smart_resize(256, 256, 32, 56 * 56, 10 ** 6) == (256, 256)
    h, w = V.smart_resize(3000, 2000, 32, 56 * 56, 512 * 512)
    assert h % 32 == 0 and w % 32 == 0 and h * w <= 512 * 512 and abs(h / w - 1.5) < 0.1
    h, w = V.smart_resize(10, 20, 32, 56 * 56, 10 ** 6)
    assert h * w >= 56 * 56
    with pytest.raises(ValueError):
        V.smart_resize(10, 5000, 32, 1, 10 ** 9)


def test_preprocess_and_tower_shapes():
    spec = V.tiny_vision(out_hidden=96)
    img = png.decode_png(png.encode_png(96, 64, png.GREEN, box=(8, 8, 40, 40)))
    patches, grid = V.preprocess(img, spec)
    assert grid == (1, 4, 6) and patches.shape == (24, spec.patch_dim)
    # a solid region gives identical patches; normalisation maps 0..255 to -1..1
    assert patches.abs().max() <= 1.0 + 1e-5
    tower = V.VisionTower(spec)
    out = tower.forward(patches, grid)
    assert out.shape == (6, 96) and tower.n_tokens(grid) == 6 and torch.isfinite(out).all()
    # merge-window order: the first 4 patch rows are the 2 x 2 window at the top-left corner
    solid = V.preprocess(np.full((64, 64, 3), 200, np.uint8), spec)[0]
    assert torch.allclose(solid[0], solid[5])
    # different pixels -> different embeddings; same pixels -> same embeddings
    other = tower.forward(*V.preprocess(png.decode_png(png.encode_png(96, 64, png.RED)), spec))
    assert not torch.allclose(out, other)
    assert torch.equal(out, tower.forward(patches, grid))


def test_scatter_and_mrope_positions():
    pad = 7
    ids = [1, 2, pad, pad, pad, pad, pad, pad, 3, 4]
    emb = torch.zeros(10, 4)
    img = torch.arange(24, dtype=torch.float32).view(6, 4)
    V.scatter_images(emb, torch.tensor(ids), pad, [img])
    assert torch.equal(emb[2:8], img) and emb[:2].abs().sum() == 0
    pos, nxt = V.mrope_positions(ids, pad, [(1, 4, 6)])
    assert pos[:, :2].tolist() == [[0, 1]] * 3
    assert pos[0, 2:8].tolist() == [2] * 6
    assert pos[1, 2:8].tolist() == [2, 2, 2, 3, 3, 3] and pos[2, 2:8].tolist() == [2, 3, 4, 2, 3, 4]
    assert pos[:, 8].tolist() == [5, 5, 5] and nxt == 7
    with pytest.raises(ValueError):
        V.scatter_images(torch.zeros(10, 4), torch.tensor(ids), pad, [img[:5]])


def test_image_cache_by_content():
    spec = V.tiny_vision(out_hidden=32)
    tower, cache = V.VisionTower(spec), V.ImageCache(cap=2)
    a, b, c = (png.encode_png(64, 64, col) for col in (png.RED, png.GREEN, png.BLUE))
    e1, g1, f1 = cache.get(tower, a, png.decode_png)
    e2, _, f2 = cache.get(tower, a, png.decode_png)
    assert f1 == f2 and e1 is e2 and cache.hits == 1
    cache.get(tower, b, png.decode_png); cache.get(tower, c, png.decode_png)
    assert len(cache.items) == 2 and f1 not in cache.items
