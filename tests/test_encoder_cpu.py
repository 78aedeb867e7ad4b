"""BERT-family encoder embeddings: hidden states against transformers, and the embeddings-only server."""
import tempfile

import pytest
import torch
from fastapi.testclient import TestClient

transformers = pytest.importorskip("transformers")

from mlxcel_b200.models.encoder import BertEncoder  # noqa: E402
from mlxcel_b200.server.embeddings import create_embedding_app  # noqa: E402
from mlxcel_b200.tokenizer import ByteTokenizer  # noqa: E402


def _tiny_bert():
    from transformers import BertConfig, BertModel
    torch.manual_seed(0)
    m = BertModel(BertConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
                             vocab_size=300, max_position_embeddings=64)).float().eval()
    with torch.no_grad():
        for _, p in m.named_parameters():
            if p.dim() >= 2:
                p.normal_(0, 0.08)
            else:
                p.add_(torch.randn_like(p) * 0.1)
    d = tempfile.mkdtemp(prefix="bert_")
    m.save_pretrained(d, safe_serialization=True)
    return m, d


def test_bert_hidden_states_match_transformers():
    m, d = _tiny_bert()
    ids = torch.randint(0, 300, (19,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = m(ids[None]).last_hidden_state[0]
    enc = BertEncoder.from_pretrained(d, dtype=torch.float32)
    got = enc.hidden_states(ids.tolist())
    assert (got - want).abs().max().item() < 1e-4
    v = enc.embed(ids.tolist(), "cls")
    assert abs(v.norm().item() - 1.0) < 1e-5 and torch.allclose(v, want[0] / want[0].norm(), atol=1e-5)


def test_embedding_server_routes():
    _, d = _tiny_bert()
    enc = BertEncoder.from_pretrained(d, dtype=torch.float32)
    app = create_embedding_app(enc, ByteTokenizer(300), "tiny-bert", api_keys={"k"})
    with TestClient(app) as c:
        assert c.post("/v1/embeddings", json=dict(input="hi")).status_code == 401
        h = {"authorization": "Bearer k"}
        r = c.post("/v1/embeddings", json=dict(input=["hello", "world!"]), headers=h).json()
        assert len(r["data"]) == 2 and len(r["data"][0]["embedding"]) == 64 and r["usage"]["prompt_tokens"] > 0
        one = c.post("/embedding", json=dict(content="hello"), headers=h).json()
        assert one[0]["embedding"] == pytest.approx(r["data"][0]["embedding"], abs=1e-6)
        assert c.get("/v1/models", headers=h).json()["data"][0]["id"] == "tiny-bert"


def test_modernbert_hidden_states_match_transformers():
    from transformers import ModernBertConfig, ModernBertModel

    from mlxcel_b200.models.encoder import ModernBertEncoder, load_encoder

    torch.manual_seed(0)
    m = ModernBertModel(ModernBertConfig(hidden_size=64, intermediate_size=96, num_hidden_layers=4, num_attention_heads=4,
                                         vocab_size=300, max_position_embeddings=128, local_attention=8,
                                         global_attn_every_n_layers=3, pad_token_id=0)).float().eval()
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() >= 2:
                p.normal_(0, 0.08)
            else:
                p.add_(torch.randn_like(p) * 0.1)
    d = tempfile.mkdtemp()
    m.save_pretrained(d)
    ids = torch.randint(1, 300, (29,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = m(ids[None]).last_hidden_state[0]
    enc = load_encoder(d, dtype=torch.float32)
    assert isinstance(enc, ModernBertEncoder) and any(enc.local) and not all(enc.local)
    got = enc.hidden_states(ids.tolist())
    assert (got - want).abs().max().item() < 2e-5 * max(1.0, want.abs().max().item())
    e = enc.embed(ids.tolist())
    assert abs(e.norm().item() - 1.0) < 1e-5


def test_embed_cli_prints_vectors_and_cosine(capsys):
    import json

    from mlxcel_b200 import cli

    _, d = _tiny_bert()
    cli.main(["embed", "-m", d, "--device", "cpu", "-p", "hello there", "-p", "general kenobi", "--json",
              "--dimensions", "32"])
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert len(out["embeddings"]) == 2 and len(out["embeddings"][0]) == 32
    assert abs(sum(x * x for x in out["embeddings"][0]) - 1.0) < 1e-4
    assert abs(out["cosine"][0][0] - 1.0) < 1e-5 and abs(out["cosine"][0][1] - out["cosine"][1][0]) < 1e-6


def _randomise(m):
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() >= 2:
                p.normal_(0, 0.08)
            else:
                p.add_(torch.randn_like(p) * 0.1)
    return m.float().eval()


_BERT = dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128, vocab_size=300,
             max_position_embeddings=64)


def test_cross_encoder_head_matches_transformers_and_reranks(capsys):
    import json

    from transformers import BertConfig, BertForSequenceClassification

    from mlxcel_b200 import cli
    from mlxcel_b200.models.encoder import load_encoder
    from mlxcel_b200.server.embeddings import pair_ids, rerank_scores

    torch.manual_seed(0)
    m = _randomise(BertForSequenceClassification(BertConfig(num_labels=1, **_BERT)))
    d = tempfile.mkdtemp()
    m.save_pretrained(d)
    ids = torch.randint(1, 300, (21,), generator=torch.Generator().manual_seed(2))
    tt = torch.tensor([0] * 9 + [1] * 12)
    with torch.no_grad():
        want = m(ids[None], token_type_ids=tt[None]).logits[0]
    enc = load_encoder(d, dtype=torch.float32)
    assert (enc.sequence_logits(ids.tolist(), tt.tolist()) - want).abs().max().item() < 1e-5
    tok = ByteTokenizer()
    pi, pt = pair_ids(tok, "query", "a document", 64)
    assert len(pi) == len(pt) and pt[0] == 0 and pt[-1] == 1
    scores = rerank_scores(enc, tok, "query", ["doc one", "another"])
    assert len(scores) == 2 and all(0.0 < s < 1.0 for s in scores)
    cli.main(["rerank", "-m", d, "--device", "cpu", "-q", "query", "-d", "doc one", "-d", "another", "--json"])
    res = json.loads(capsys.readouterr().out.strip().splitlines()[-1])["results"]
    assert [r["index"] for r in res] == sorted(range(2), key=lambda i: -scores[i])
    app = create_embedding_app(enc, tok, "ce")
    r = TestClient(app).post("/v1/rerank", json=dict(query="query", documents=["doc one", "another"], top_n=1))
    assert r.status_code == 200 and len(r.json()["results"]) == 1


def test_token_classification_head_and_tagging():
    from transformers import BertConfig, BertForTokenClassification

    from mlxcel_b200.models.encoder import bio_spans, load_encoder
    from mlxcel_b200.server.embeddings import tag_text

    labels = {0: "O", 1: "B-PER", 2: "I-PER", 3: "B-LOC", 4: "I-LOC"}
    torch.manual_seed(0)
    m = _randomise(BertForTokenClassification(BertConfig(num_labels=5, id2label=labels,
                                                         label2id={v: k for k, v in labels.items()}, **_BERT)))
    d = tempfile.mkdtemp()
    m.save_pretrained(d)
    ids = torch.randint(1, 300, (17,), generator=torch.Generator().manual_seed(3))
    with torch.no_grad():
        want = m(ids[None]).logits[0]
    enc = load_encoder(d, dtype=torch.float32)
    assert enc.token_head and (enc.token_logits(ids.tolist()) - want).abs().max().item() < 1e-5
    assert bio_spans(["O", "B-PER", "I-PER", "O", "I-LOC", "B-LOC", "B-LOC", "I-LOC"]) == \
        [(1, 3, "PER"), (4, 5, "LOC"), (5, 6, "LOC"), (6, 8, "LOC")]
    assert bio_spans(["S-X", "B-Y", "E-Y"]) == [(0, 1, "X"), (1, 3, "Y")]
    res = tag_text(enc, ByteTokenizer(), "Sarah lives in Paris", keep=None, replacement="#")
    assert isinstance(res["redacted"], str) and all(s["end_token"] > s["start_token"] for s in res["spans"])
    with pytest.raises(ValueError):
        enc.sequence_logits(ids.tolist())


def test_sentence_transformers_pooling_defaults_and_maxsim(tmp_path, capsys):
    import json
    import shutil

    from mlxcel_b200 import cli
    from mlxcel_b200.models.encoder import load_encoder, maxsim

    _, d = _tiny_bert()
    st = tmp_path / "st"
    shutil.copytree(d, st)
    (st / "1_Pooling").mkdir()
    (st / "1_Pooling" / "config.json").write_text(json.dumps(dict(pooling_mode_cls_token=True, pooling_mode_mean_tokens=False)))
    (st / "modules.json").write_text(json.dumps([dict(idx=0, type="sentence_transformers.models.Transformer"),
                                                 dict(idx=1, type="sentence_transformers.models.Pooling")]))
    enc = load_encoder(str(st), dtype=torch.float32)
    assert (enc.default_pooling, enc.default_normalize) == ("cls", False)
    plain = load_encoder(d, dtype=torch.float32)
    assert (plain.default_pooling, plain.default_normalize) == ("mean", True)
    cli.main(["embed", "-m", str(st), "--device", "cpu", "-p", "hello", "--json"])
    v = torch.tensor(json.loads(capsys.readouterr().out.strip().splitlines()[-1])["embeddings"][0])
    ids = ByteTokenizer().encode("hello", add_special_tokens=True)
    want = load_encoder(str(st)).hidden_states(ids)[0].float()           # [CLS] state, not normalised
    assert torch.allclose(v, want, atol=1e-5) and abs(v.norm().item() - 1.0) > 1e-3
    q, doc = enc.hidden_states([5, 6, 7]), enc.hidden_states([5, 6, 7, 8, 9])
    assert abs(maxsim(q, q) - 3.0) < 1e-4 and maxsim(q, doc) <= 3.0 + 1e-5


def test_bio_viterbi_repairs_invalid_paths():
    from mlxcel_b200.models.encoder import bio_viterbi

    labels = ["O", "B-PER", "I-PER", "B-LOC", "I-LOC"]
    lp = torch.full((4, 5), -5.0)
    lp[0, 0] = lp[1, 2] = lp[2, 2] = lp[3, 0] = -0.1           # argmax path O I-PER I-PER O is invalid
    lp[1, 1] = -0.5                                            # B-PER is the cheap repair at position 1
    assert [labels[i] for i in bio_viterbi(lp, labels)] == ["O", "B-PER", "I-PER", "O"]
    lp2 = torch.full((3, 5), -5.0)
    lp2[0, 1] = lp2[1, 4] = lp2[2, 0] = -0.1                   # B-PER then I-LOC: entity mismatch
    lp2[1, 2] = -0.3
    assert [labels[i] for i in bio_viterbi(lp2, labels)] == ["B-PER", "I-PER", "O"]
    valid = torch.full((3, 5), -5.0)
    valid[0, 3] = valid[1, 4] = valid[2, 0] = -0.1
    assert [labels[i] for i in bio_viterbi(valid, labels)] == ["B-LOC", "I-LOC", "O"]
    bioes = ["O", "B-X", "I-X", "E-X", "S-X"]
    e = torch.full((3, 5), -5.0)
    e[0, 1] = e[1, 0] = e[2, 0] = -0.1                         # B-X followed by O: an entity left open
    e[1, 2] = e[2, 3] = -0.4
    assert [bioes[i] for i in bio_viterbi(e, bioes)] in (["B-X", "I-X", "E-X"], ["S-X", "O", "O"], ["O", "O", "O"])
    assert bioes[bio_viterbi(e, bioes)[-1]] not in ("B-X", "I-X")


@pytest.mark.parametrize("share,buckets", [(True, 8), (False, -1)])
def test_deberta_v2_matches_transformers(share, buckets):
    """Disentangled attention (content-to-position and position-to-content terms over log-bucketed
    relative positions, shared or dedicated positional projections) and the cross-encoder head."""
    import tempfile

    from transformers import DebertaV2Config, DebertaV2ForSequenceClassification

    from mlxcel_b200.models.encoder import load_encoder
    torch.manual_seed(0)
    hc = DebertaV2Config(vocab_size=300, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
                         max_position_embeddings=64, relative_attention=True, pos_att_type=["p2c", "c2p"],
                         share_att_key=share, position_buckets=buckets, norm_rel_ebd="layer_norm",
                         position_biased_input=False, max_relative_positions=-1 if buckets > 0 else 32, num_labels=1)
    m = DebertaV2ForSequenceClassification(hc).eval()
    d = tempfile.mkdtemp(prefix="deberta_")
    m.save_pretrained(d, safe_serialization=True)
    enc = load_encoder(d, dtype=torch.float32)
    ids = torch.randint(0, 300, (1, 37), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = m.deberta(ids).last_hidden_state[0]
        want_logit = m(ids).logits[0]
    assert (enc.hidden_states(ids[0].tolist()) - want).abs().max().item() < 1e-4
    assert (enc.classify(ids[0].tolist()) - want_logit).abs().max().item() < 1e-4
    v = enc.embed(ids[0].tolist())
    assert abs(float(v.norm()) - 1.0) < 1e-5


def test_siglip_text_tower_matches_transformers(tmp_path):
    """SigLIP text encoder, from a text-only checkpoint and from the text half of a full SigLIP
    checkpoint: final hidden states and the pooled sentence vector (head over the last token)."""
    from transformers import SiglipConfig, SiglipModel, SiglipTextConfig, SiglipTextModel

    from mlxcel_b200.models.encoder import SiglipTextEncoder, load_encoder

    torch.manual_seed(0)
    tc = dict(vocab_size=120, hidden_size=48, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
              max_position_embeddings=16)
    ids = [5, 17, 99, 3, 42, 7, 1]
    text = SiglipTextModel(SiglipTextConfig(**tc)).float().eval()
    full = SiglipModel(SiglipConfig(text_config=tc, vision_config=dict(hidden_size=32, intermediate_size=64, num_hidden_layers=1,
                                                                       num_attention_heads=2, image_size=16, patch_size=8))).float().eval()
    for name, model, tower in (("text", text, text.text_model), ("full", full, full.text_model)):
        with torch.no_grad():
            for p in model.parameters():
                if p.dim() >= 2:
                    p.normal_(0, 0.1)
                else:
                    p.add_(torch.randn_like(p) * 0.1)
            out = tower(input_ids=torch.tensor([ids]))
        d = tmp_path / name
        model.save_pretrained(d, safe_serialization=True)
        enc = load_encoder(d, dtype=torch.float32)
        assert isinstance(enc, SiglipTextEncoder) and enc.default_pooling == "last"
        assert (enc.hidden_states(ids) - out.last_hidden_state[0]).abs().max() < 2e-4
        assert (enc.embed(ids, "last", normalize=False) - out.pooler_output[0]).abs().max() < 2e-4
        v = enc.embed(ids)
        assert abs(float(v.norm()) - 1.0) < 1e-5
