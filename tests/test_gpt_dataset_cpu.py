"""GPT samples from indexed datasets: packing, determinism, splits, blending, Megatron index format, --data-path training."""
import os
import struct
import sys
import tempfile

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _corpus(prefix, n_docs=40, seed=0, vocab=200, eod=1):
    from mindspeed_b200.data_tools.indexed_dataset import IndexedDatasetBuilder
    rs = np.random.RandomState(seed)
    b = IndexedDatasetBuilder(prefix, dtype=np.uint16)
    docs = []
    for _ in range(n_docs):
        d = list(rs.randint(2, vocab, size=rs.randint(5, 60))) + [eod]
        docs.append(d)
        b.add_item(d)
        b.end_document()
    b.finalize()
    return docs


def test_samples_pack_the_whole_stream_once_per_epoch():
    from mindspeed_b200.data_tools.indexed_dataset import MMapIndexedDataset
    from mindspeed_b200.training.gpt_dataset import GPTDataset
    with tempfile.TemporaryDirectory() as d:
        docs = _corpus(os.path.join(d, "c"))
        ix = MMapIndexedDataset(os.path.join(d, "c"))
        ds = GPTDataset(ix, (0, len(docs)), seq_length=16, seed=3, eod_token=1, reset_position_ids=True, eod_mask_loss=True)
        total = sum(len(x) for x in docs)
        assert ds.samples_per_epoch == (total - 1) // 16
        # every epoch-0 sample is a window of the shuffled-document stream; together they cover its first n*16 tokens once
        order, cum, shuffle = ds._epoch(0)
        stream = np.concatenate([np.asarray(docs[int(k)]) for k in order])
        seen = np.zeros(ds.samples_per_epoch, dtype=bool)
        for i in range(ds.samples_per_epoch):
            t = ds.tokens_of(i)
            w = int(shuffle[i])
            assert np.array_equal(t, stream[w * 16:w * 16 + 17])
            seen[w] = True
        assert seen.all()
        # same index, same sample; another epoch, another order
        assert np.array_equal(ds.tokens_of(5), ds.tokens_of(5))
        assert not np.array_equal(ds._epoch(0)[0], ds._epoch(1)[0])
        it = ds[2]
        assert torch.equal(it["tokens"][1:], it["labels"][:-1])
        eod = it["tokens"] == 1
        assert (it["loss_mask"][eod] == 0).all() and (it["loss_mask"][~eod] == 1).all()
        # positions restart after an end-of-document token
        pos = it["position_ids"]
        for j in range(1, 16):
            assert pos[j] == (0 if it["tokens"][j - 1] == 1 else pos[j - 1] + 1)


def test_split_blend_and_megatron_index_format():
    from mindspeed_b200.data_tools.indexed_dataset import MMapIndexedDataset
    from mindspeed_b200.training.gpt_dataset import build_train_valid_test_datasets, split_documents
    assert split_documents(100, "90,5,5") == [(0, 90), (90, 95), (95, 100)]
    assert split_documents(10, "100,0,0") == [(0, 10), (10, 10), (10, 10)]
    with tempfile.TemporaryDirectory() as d:
        _corpus(os.path.join(d, "a"), seed=1)
        _corpus(os.path.join(d, "b"), seed=2)
        tr, va, te = build_train_valid_test_datasets([os.path.join(d, "a")], "80,10,10", 8, 7)
        assert tr is not None and va is not None and te is not None and len(tr) > len(va)
        bl, _, _ = build_train_valid_test_datasets(["3", os.path.join(d, "a"), "1", os.path.join(d, "b")], "100,0,0", 8, 7, (400, None, None))
        assert len(bl) == 400
        share = (bl.which[:100] == 0).mean()
        assert abs(share - 0.75) < 0.02
        assert bl[0]["tokens"].shape == (8,)
        # the same corpus with a Megatron-style index header is read identically
        own = MMapIndexedDataset(os.path.join(d, "a"))
        with open(os.path.join(d, "m.idx"), "wb") as f:
            f.write(b"MMIDIDX\x00\x00")
            f.write(struct.pack("<QBQQ", 1, 8, len(own.lengths), len(own.doc_idx)))       # 8 = uint16 in that format
            f.write(np.asarray(own.lengths, dtype=np.int32).tobytes())
            f.write(np.asarray(own.offsets, dtype=np.int64).tobytes())
            f.write(np.asarray(own.doc_idx, dtype=np.int64).tobytes())
        with open(os.path.join(d, "a.bin"), "rb") as src, open(os.path.join(d, "m.bin"), "wb") as dst:
            dst.write(src.read())
        meg = MMapIndexedDataset(os.path.join(d, "m"))
        assert len(meg) == len(own) and all(np.array_equal(meg[i], own[i]) for i in range(len(own)))


def _train_on_files(rank, world, prefix):
    import io
    from contextlib import redirect_stdout
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import pretrain_gpt as pg
    from test_pipeline_cpu import BASE
    from mindspeed_b200.training import pretrain
    with redirect_stdout(io.StringIO()):
        hist = pretrain(pg.train_valid_test_datasets_provider, pg.model_provider, forward_step_func=pg.forward_step,
                        args_list=BASE + ["--data-path", prefix, "--split", "100,0,0", "--eod-mask-loss", "--train-iters", "6",
                                          "--lr", "5e-3"])
    return [h["lm loss"] for h in hist]


def test_pretrain_reads_data_path():
    from dist_utils import run_distributed
    with tempfile.TemporaryDirectory() as d:
        _corpus(os.path.join(d, "c"), n_docs=120, vocab=100)
        losses = run_distributed(_train_on_files, 2, os.path.join(d, "c"))[0]
        assert len(losses) == 6 and losses[-1] < losses[0]


def test_varlen_attention_matches_document_mask():
    from mindspeed_b200.ops.attention import attention_ref, varlen_attention
    torch.manual_seed(0)
    s, n, d = 24, 2, 8
    q, k, v = (torch.randn(s, 1, n, d, requires_grad=True) for _ in range(3))
    cu = [0, 5, 6, 17, 24]
    doc = torch.zeros(s, dtype=torch.long)
    for i, (a, b) in enumerate(zip(cu[:-1], cu[1:])):
        doc[a:b] = i
    masked = ~(torch.tril(torch.ones(s, s, dtype=torch.bool)) & (doc.view(-1, 1) == doc.view(1, -1)))
    ref = attention_ref(q, k, v, causal=False, mask=masked.view(1, 1, s, s))
    w = torch.randn_like(ref)
    gr = torch.autograd.grad((ref * w).sum(), (q, k, v))
    out = varlen_attention(q, k, v, cu, causal=True)
    gg = torch.autograd.grad((out * w).sum(), (q, k, v))
    torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5)
    for a, b in zip(gg, gr):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-5)


def _train_packed(rank, world, prefix, extra):
    import io
    from contextlib import redirect_stdout
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import pretrain_gpt as pg
    from test_pipeline_cpu import BASE
    from mindspeed_b200.models import attention as MA
    from mindspeed_b200.ops import attention as OA
    from mindspeed_b200.training import pretrain
    calls = {"n": 0, "docs": 0}
    orig = OA.varlen_attention

    def counted(q, k, v, cu, *a, **kw):
        calls["n"] += 1
        calls["docs"] += len(cu) - 1
        return orig(q, k, v, cu, *a, **kw)
    OA.varlen_attention = counted
    with redirect_stdout(io.StringIO()):
        hist = pretrain(pg.train_valid_test_datasets_provider, pg.model_provider, forward_step_func=pg.forward_step,
                        args_list=BASE + ["--data-path", prefix, "--split", "100,0,0", "--train-iters", "3", "--tokenizer-type",
                                          "NullTokenizer", "--vocab-size", "127", "--make-vocab-size-divisible-by", "128"] + list(extra))
    return [h["lm loss"] for h in hist], calls


def test_training_with_reset_attention_mask_uses_packed_attention():
    """--reset-attention-mask --reset-position-ids: attention runs per document (and the rotary positions restart), which
    changes the loss relative to attending across documents."""
    from dist_utils import run_distributed
    with tempfile.TemporaryDirectory() as d:
        # NullTokenizer(vocab 127): eod id 127 -> the corpus closes documents with 127; the model's vocabulary is 128
        _corpus(os.path.join(d, "c"), n_docs=80, vocab=100, eod=127)
        plain, c0 = run_distributed(_train_packed, 1, os.path.join(d, "c"), [])[0]
        packed, c1 = run_distributed(_train_packed, 1, os.path.join(d, "c"), ["--reset-attention-mask", "--reset-position-ids",
                                                                              "--eod-mask-loss"])[0]
        assert c0["n"] == 0 and c1["n"] > 0 and c1["docs"] > c1["n"]          # several documents per sample
        assert plain != packed and all(abs(a - b) < 0.5 for a, b in zip(plain, packed))


def test_equal_sub_sequences_fold_into_the_batch_axis():
    from mindspeed_b200.ops.attention import attention_ref, varlen_attention
    from mindspeed_b200.training.data import fixed_sub_seq_boundaries
    assert fixed_sub_seq_boundaries(32, 8) == [0, 8, 16, 24, 32]
    assert fixed_sub_seq_boundaries(30, 8) == [0, 8, 16, 24, 30]
    assert fixed_sub_seq_boundaries(8, 8) == [0, 8]
    torch.manual_seed(0)
    s, b, n, d = 32, 3, 2, 8
    q, k, v = (torch.randn(s, b, n, d, requires_grad=True) for _ in range(3))
    for cu in ([0, 8, 16, 24, 32], [0, 12, 24, 32]):                 # folded path / one call per sub-sequence, batch of 3
        doc = torch.zeros(s, dtype=torch.long)
        for i, (a, e) in enumerate(zip(cu[:-1], cu[1:])):
            doc[a:e] = i
        masked = ~(torch.tril(torch.ones(s, s, dtype=torch.bool)) & (doc.view(-1, 1) == doc.view(1, -1)))
        ref = attention_ref(q, k, v, causal=False, mask=masked.view(1, 1, s, s))
        out = varlen_attention(q, k, v, cu, causal=True)
        w = torch.randn_like(ref)
        torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5)
        for a, e in zip(torch.autograd.grad((out * w).sum(), (q, k, v)), torch.autograd.grad((ref * w).sum(), (q, k, v))):
            torch.testing.assert_close(a, e, rtol=1e-5, atol=1e-5)


def _train_fixed(rank, world, extra):
    import io
    from contextlib import redirect_stdout
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import pretrain_gpt as pg
    from test_pipeline_cpu import BASE
    from mindspeed_b200.training import pretrain
    seen = []
    orig = pg.get_batch

    def spy(*a, **kw):
        out = orig(*a, **kw)
        seen.append((out[5], out[4][:, :12].tolist()))
        return out
    pg.get_batch = spy
    base = list(BASE)
    base[base.index("--micro-batch-size") + 1] = "2"
    with redirect_stdout(io.StringIO()):
        hist = pretrain(pg.train_valid_test_datasets_provider, pg.model_provider, forward_step_func=pg.forward_step,
                        args_list=base + list(extra))
    pg.get_batch = orig
    return [h["lm loss"] for h in hist], seen[0]


def test_fixed_sub_sequence_length_sets_boundaries_and_positions_for_any_batch():
    """--reset-attention-mask --fix-sub-seq-length 8 on synthetic data with micro-batch 2: attention and rotary positions
    restart every 8 tokens (sequence length 32 -> four sub-sequences per row)."""
    from dist_utils import run_distributed
    plain, (p0, _) = run_distributed(_train_fixed, 1, [])[0]
    fixed, (p1, pos) = run_distributed(_train_fixed, 1, ["--reset-attention-mask", "--fix-sub-seq-length", "8"])[0]
    assert p0 is None and p1["cu_seqlens"] == [0, 8, 16, 24, 32]
    assert pos == [[0, 1, 2, 3, 4, 5, 6, 7, 0, 1, 2, 3]] * 2
    assert plain != fixed and all(abs(a - b) < 0.5 for a, b in zip(plain, fixed))
    # a sub-sequence length above the sequence length leaves the documents' own boundaries (none here): refused without data
    from mindspeed_b200.training.arguments import parse_args, validate_args
    with pytest.raises(AssertionError, match="data-path"):
        validate_args(parse_args(args_list=["--num-layers", "2", "--hidden-size", "64", "--num-attention-heads", "4", "--seq-length",
                                            "32", "--micro-batch-size", "1", "--vocab-size", "128", "--reset-attention-mask",
                                            "--fix-sub-seq-length", "64"]))
