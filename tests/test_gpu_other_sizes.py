"""The engine at sizes that the family's own checkpoints do not have: head sizes of 80, 96, 112,
160, 192 and 256 (every step of 16 is allowed), groups of 5, 7 and 8 query heads, one key/value
head and as many as query heads, widths and feed-forward widths that are no multiple of 8, odd
vocabularies, other pages, eps and rope constants.  Each configuration under the four cuts, in
32-bit and in bfloat16, against the plain implementation; attention peaked (tiny_configs.sharp),
so that a key that is lost or read from the wrong place shows."""
import pytest

import replay_util as ru
from helpers import load_plain, random_tokens
from tiny_configs import sharp

pytestmark = pytest.mark.gpu


def _llama(hd, n_q, n_kv, d, ff, vocab, layers, eps=1e-5, theta=10000.0, scaling=None, tied=True):
    return {"architectures": ["LlamaForCausalLM"], "hidden_size": d, "intermediate_size": ff,
            "num_hidden_layers": layers, "num_attention_heads": n_q, "num_key_value_heads": n_kv,
            "head_dim": hd, "vocab_size": vocab, "max_position_embeddings": 4096, "rms_norm_eps": eps,
            "rope_theta": theta, "rope_scaling": scaling, "tie_word_embeddings": tied, "hidden_act": "silu"}


def _llama3(factor, high, original):
    return {"rope_type": "llama3", "factor": factor, "low_freq_factor": 1.0, "high_freq_factor": high,
            "original_max_position_embeddings": original}


# name: (config.json, page size, request lengths)
SIZES = {
    "hd80_groups_of_5": (_llama(80, 10, 2, 136, 344, 999, 2, eps=3e-4, theta=1234.5,
                                scaling=_llama3(3.5, 2.5, 100), tied=False), 16, [77, 126, 300, 45]),
    "hd96_as_many_kv_heads": (_llama(96, 7, 7, 200, 150, 331, 1), 8, [40, 203, 66]),
    "hd112_one_kv_head": (_llama(112, 8, 1, 72, 520, 2049, 3, eps=1e-6, theta=500000.0,
                                 scaling=_llama3(8.0, 4.0, 256)), 32, [150, 35, 410, 90]),
    "hd160_width_not_of_8": (_llama(160, 6, 3, 90, 198, 1024, 2, tied=False), 16, [186, 88, 361, 66]),
    "hd192_groups_of_5": (_llama(192, 5, 1, 256, 100, 4099, 1, theta=500000.0,
                                 scaling=_llama3(32.0, 4.0, 64), tied=False), 64, [45, 174, 477]),
    "hd256": (_llama(256, 4, 2, 64, 104, 1220, 2), 8, [93, 70, 259]),
    "hd64_groups_of_7": (_llama(64, 21, 3, 154, 758, 1373, 2, eps=1e-6), 16, [52, 345, 260, 39, 71]),
}
CUTS = {"whole": ru.whole, "tail": ru.tail_by_token, "ragged": ru.ragged, "mixed": ru.mixed}


@pytest.fixture(scope="module")
def made(tmp_path_factory):
    """{name: (folder, config dictionary, requests, plain logits)}, each made when first asked for."""
    from nanoinfer_b200.weights import write_random_model
    root, cache = tmp_path_factory.mktemp("other_sizes"), {}

    def get(name):
        if name not in cache:
            raw, page, lens = SIZES[name]
            folder = str(root / name)
            write_random_model(folder, raw, seed=len(name), slot_std=sharp(raw))
            raw_read, weights = load_plain(folder)
            reqs = {f"r{i}": random_tokens(raw["vocab_size"], n, 7000 + 10 * len(name) + i) for i, n in enumerate(lens)}
            cache[name] = (folder, raw_read, reqs, ru.plain_logits(raw_read, weights, reqs))
        return cache[name]
    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("name", list(SIZES))
def test_other_sizes_match_plain(made, name, cut, dtype):
    from nanoinfer_b200.config import load_config
    from nanoinfer_b200.engine import ModelRunner
    from nanoinfer_b200.kernels import ops
    from nanoinfer_b200.weights import load_weights
    folder, raw, reqs, want = made(name)
    page = SIZES[name][1]
    steps = CUTS[cut](reqs)
    cfg = load_config(folder)
    # exactly the pages the trace needs at its fullest (requests rounded up to 64 or to a page)
    num_pages = -(-ru.max_live_tokens(steps, max(64, page)) // page)
    runner = ModelRunner(cfg, load_weights(folder, cfg), dtype=dtype, page_size=page, num_pages=num_pages,
                         max_requests=4)
    got = ru.run_trace(runner, steps)
    ops.check_device_errors()
    assert len(got) == sum(len(t) for t in reqs.values())
    ru.compare(got, want, dtype, label=f"{name}/{cut}/{dtype}")
    runner.cache.check_consistency()
    assert runner.cache.num_free_pages(0) == runner.cache.pools[0].num_pages
