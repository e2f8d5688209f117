"""Tile-shape selection (the counterpart of the reference's dead autotuner, src/autotune_sa.cpp):
the cache and the random-step search are host logic and are tested without a device; the search on
the device is a GPU test."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cache_round_trips_through_a_file(cake, tmp_path):
    cake.tune_clear()
    assert cake.tune_get(3000, 3000, 3000, cake.MKN) is None
    cake.tune_put(3000, 3000, 3000, cake.MKN, 256, 4, 2, 0.25)
    cake.tune_put(1024, 65536, 1024, cake.NKM, 128, 16, 0, 0.5)
    path = tmp_path / "tune.json"
    assert cake.tune_save(path) == 2
    text = json.loads(path.read_text())  # the file is JSON
    assert text["version"] == 2 and len(text["entries"]) == 2
    assert all(e["cluster"] == 0 for e in text["entries"])  # the cluster shape was left to the rule
    cake.tune_clear()
    assert cake.tune_get(3000, 3000, 3000, cake.MKN) is None
    assert cake.tune_load(path) == 2
    got = cake.tune_get(3000, 3000, 3000, cake.MKN)
    assert (got["tile_n"], got["band"], got["k_pieces"]) == (256, 4, 2) and abs(got["ms"] - 0.25) < 1e-6
    assert cake.tune_get(1024, 65536, 1024, cake.NKM)["band"] == 16
    assert cake.tune_get(3000, 3000, 3000, cake.KMN) is None  # the schedule is part of the key
    with pytest.raises(cake.CakeError):
        cake.tune_put(10, 10, 10, cake.KMN, 192, 8, 0)  # not a tile width
    with pytest.raises(cake.CakeError):
        cake.tune_load(tmp_path / "missing.json")
    cake.tune_clear()


def test_environment_file_is_loaded_on_first_use(cake, tmp_path):
    path = tmp_path / "env_tune.json"
    cake.tune_clear()
    cake.tune_put(2048, 2048, 2048, cake.KMN, 128, 8, 3, 0.1)
    cake.tune_save(path)
    cake.tune_clear()
    code = ("import cake_on_cpu_b200 as c; e = c.tune_get(2048, 2048, 2048, c.KMN); "
            "print(e['tile_n'], e['band'], e['k_pieces'])")
    env = dict(os.environ, CAKE_AUTOTUNE_CACHE=str(path), PYTHONPATH=ROOT)
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True)
    assert out.stdout.split() == ["128", "8", "3"], out.stderr


def test_random_step_search_finds_the_cheapest_point(cake):
    """The search never evaluates a point twice, starts from the rule's choice and, given enough trials to
    cover the grid, returns the global minimum of an arbitrary cost."""
    seen = []

    def cost(tile_n, band, k_pieces):
        seen.append((tile_n, band, k_pieces))
        if k_pieces == 12:
            return -1.0  # an invalid point is skipped
        return 1.0 + abs(tile_n - 128) / 128.0 + abs(band - 4) * 0.1 + abs(k_pieces - 3) * 0.05

    got = cake.tune_search(4096, 4096, 4096, cost, trials=200, seed=7)
    assert len(seen) == len(set(seen)) == got["evaluated"]
    assert seen[0] == (256, 8, 0)  # the rule: wide tile, bands of 8, the library's own cut
    assert (got["tile_n"], got["band"], got["k_pieces"]) == (128, 4, 3) and abs(got["ms"] - 1.0) < 1e-6
    # a short search still returns the best point it saw
    seen.clear()
    got = cake.tune_search(4096, 4096, 4096, cost, trials=6, seed=3)
    assert got["evaluated"] == 6 and len(seen) == 6
    assert got["ms"] == pytest.approx(min(cost(*p) for p in list(seen) if p[2] != 12))
    # narrow products have one tile width only
    seen.clear()
    cake.tune_search(4096, 100, 4096, cost, trials=500)
    assert {w for w, _, _ in seen} == {128}


def test_cluster_shape_is_part_of_an_entry_and_of_the_search(cake, tmp_path):
    """The cluster shape (1 = the two CTAs of a cluster on a 256-row tile, 2 = one CTA per 128-row tile) is recorded
    with the tile shape, survives the file, defaults to the rule (0) in a file written without it, and is an axis
    of the search."""
    cake.tune_clear()
    cake.tune_put(8192, 8192, 8192, cake.KMN, 256, 8, 0, 3.6, cluster=1)
    cake.tune_put(300, 4096, 4096, cake.MKN, 256, 8, 2, 0.1, cluster=2)
    assert cake.tune_get(8192, 8192, 8192, cake.KMN)["cluster"] == 1
    path = tmp_path / "shapes.json"
    assert cake.tune_save(path) == 2
    cake.tune_clear()
    assert cake.tune_load(path) == 2
    assert cake.tune_get(300, 4096, 4096, cake.MKN)["cluster"] == 2
    with pytest.raises(cake.CakeError):
        cake.tune_put(10, 10, 10, cake.KMN, 128, 8, 0, cluster=3)
    old = tmp_path / "old.json"
    old.write_text('{"version": 1, "kernel": "sgemm_tf32x3", "entries": [\n'
                   '  {"M": 512, "N": 512, "K": 512, "sched": 0, "tile_n": 128, "band": 4, "k_pieces": 2, "ms": 0.020000}\n]}\n')
    cake.tune_clear()
    assert cake.tune_load(old) == 1
    got = cake.tune_get(512, 512, 512, cake.KMN)
    assert (got["tile_n"], got["cluster"], got["band"], got["k_pieces"]) == (128, 0, 4, 2)
    cake.tune_clear()

    seen = []

    def cost(tile_n, cluster, band, k_pieces):
        seen.append((tile_n, cluster, band, k_pieces))
        return 1.0 + (0.5 if cluster == 1 else 0.0) + abs(tile_n - 256) / 256.0 + abs(band - 16) * 0.01 + k_pieces * 0.01

    got = cake.tune_search_shape(4096, 4096, 4096, cost, trials=400, seed=5)
    assert len(seen) == len(set(seen)) == got["evaluated"]
    assert seen[0] == (256, 1, 8, 0)  # the rule: wide tile on pairs of SMs, bands of 8, the library's own cut
    assert (got["tile_n"], got["cluster"], got["band"], got["k_pieces"]) == (256, 2, 16, 0)
    # a single row of tiles has nothing to pair, and 300 rows would be padded to 512: the rule starts from single SMs
    seen.clear()
    cake.tune_search_shape(100, 4096, 4096, cost, trials=500)
    assert {c for _, c, _, _ in seen} == {2}
    seen.clear()
    cake.tune_search_shape(300, 4096, 4096, cost, trials=3)
    assert seen[0][1] == 2


@pytest.mark.gpu
def test_search_on_the_device_records_a_winner_that_later_products_use(cake):
    import torch
    cake.tune_clear()
    M, K, N = 3000, 1500, 2100
    g = torch.Generator(device="cuda").manual_seed(3)
    A = torch.rand((M, K), device="cuda", generator=g) * 2 - 1
    B = torch.rand((K, N), device="cuda", generator=g) * 2 - 1
    C = torch.empty((M, N), device="cuda")
    cake.cake_sgemm(A, B, C, kernel=cake.KERNEL_TF32X3)
    before = C.clone()
    entry = cake.tune(A, B, C, trials=12)
    assert entry["evaluated"] == 12 and entry["tile_n"] in (0, 128, 256) and entry["ms"] > 0  # 0: the rule was not beaten
    assert entry["cluster"] in (0, 1, 2)
    sched = cake.last_stats()["sched"]
    assert cake.tune_get(M, N, K, sched) is not None
    # the product with the tuned shape is still the product
    cake.cake_sgemm(A, B, C, kernel=cake.KERNEL_TF32X3)
    assert entry["tile_n"] == 0 or cake.last_stats()["tile_n"] == entry["tile_n"]
    exact = A[:64].double() @ B.double()
    den = A[:64].double().norm(dim=1)[:, None] * B.double().norm(dim=0)[None, :]
    assert ((C[:64].double() - exact).abs() / den).max().item() <= 1e-5
    assert ((before[:64].double() - exact).abs() / den).max().item() <= 1e-5
    # options were restored by the search
    assert [cake.get_option(k) for k in ("tile_n", "band", "k_pieces", "pair")] == [0, 0, 0, 0]
    cake.tune_clear()
