"""GPT pretraining entry point (same role and CLI shape as Megatron's pretrain_gpt.py).

  torchrun --nproc-per-node 8 --master-addr 127.0.0.1 pretrain_gpt.py --tensor-model-parallel-size 8 \
      --sequence-parallel --num-layers 32 --hidden-size 4096 ... --mock-data --optimization-level 2
"""
from functools import partial

import torch

from mindspeed_b200.models import GPTModel
from mindspeed_b200.parallel import parallel_state as ps
from mindspeed_b200.training import core_transformer_config_from_args, get_args, pretrain
from mindspeed_b200.training.data import BatchIterator, SyntheticGPTDataset, get_batch


def model_provider(pre_process=True, post_process=True):
    args = get_args()
    config = core_transformer_config_from_args(args)
    return GPTModel(config, vocab_size=args.padded_vocab_size, max_sequence_length=args.max_position_embeddings,
                    pre_process=pre_process, post_process=post_process, parallel_output=True,
                    share_embeddings_and_output_weights=not args.untie_embeddings_and_output_weights,
                    position_embedding_type=args.position_embedding_type, rotary_percent=args.rotary_percent,
                    rotary_base=args.rotary_base, rope_scaling=args.use_rope_scaling,
                    seq_len_interpolation_factor=args.rotary_seq_len_interpolation_factor)


def loss_func(loss_mask, output_tensor):
    losses = output_tensor.float()
    loss_mask = loss_mask.reshape(-1).float()
    total = torch.sum(losses.reshape(-1) * loss_mask)
    n = loss_mask.sum()
    loss = torch.stack([total, n])
    if ps.get_context_parallel_world_size() > 1:
        torch.distributed.all_reduce(loss, group=ps.get_context_parallel_group())
    rep = loss.detach().clone()
    torch.distributed.all_reduce(rep, group=ps.get_data_parallel_group())
    return loss[0] / loss[1].clamp(min=1), {"lm loss": rep}


def forward_step(data_iterator, model):
    dev = next((p.device for p in model.parameters()), None)
    if dev is None:           # a pipeline chunk made of no-op layers only holds no parameters
        on_gpu = torch.cuda.is_available() and torch.distributed.is_initialized() and torch.distributed.get_backend() != "gloo"
        dev = torch.device("cuda", torch.cuda.current_device()) if on_gpu else torch.device("cpu")
    tokens, labels, loss_mask, attention_mask, position_ids, packed = get_batch(data_iterator, dev, return_packed=True)
    args = get_args()
    if getattr(args, "qad_enable", False):
        # quantisation-aware distillation: the loss is the KL divergence from a frozen teacher's logits
        from mindspeed_b200.qat.qad import qad_forward_step
        return qad_forward_step(tokens, labels, loss_mask, attention_mask, position_ids, packed, model, args)
    out = model(tokens, position_ids, attention_mask, labels=labels, packed_seq_params=packed)
    return out, partial(loss_func, loss_mask)


def train_valid_test_datasets_provider(args):
    if getattr(args, "data_path", None):
        # indexed token datasets (this package's or Megatron's .bin / .idx); documents packed into seq_length + 1 windows
        from mindspeed_b200.training.gpt_dataset import build_train_valid_test_datasets
        n_train = args.train_iters * args.global_batch_size if args.train_iters else None
        eod = None
        if args.reset_position_ids or args.eod_mask_loss or args.reset_attention_mask:
            from mindspeed_b200.tokenizer.tokenizer import build_tokenizer
            eod = build_tokenizer(args).eod        # the end-of-document id the corpus was tokenised with
        train, _, _ = build_train_valid_test_datasets(args.data_path, args.split, args.seq_length, args.seed, (n_train, None, None),
                                                      eod_token=eod, reset_position_ids=args.reset_position_ids,
                                                      reset_attention_mask=args.reset_attention_mask, eod_mask_loss=args.eod_mask_loss)
        if train is None:
            raise ValueError("--split leaves no documents for training")
        return BatchIterator(train, args.micro_batch_size, ps.get_data_parallel_rank(), ps.get_data_parallel_world_size(),
                             start=args.iteration * args.global_batch_size, micro_batch_sizes=getattr(args, "micro_batch_sizes", None))
    ds = SyntheticGPTDataset(args.padded_vocab_size, args.seq_length, 1 << 20, seed=args.seed)
    return BatchIterator(ds, args.micro_batch_size, ps.get_data_parallel_rank(), ps.get_data_parallel_world_size(),
                         start=args.iteration * args.global_batch_size, micro_batch_sizes=getattr(args, "micro_batch_sizes", None))


if __name__ == "__main__":
    pretrain(train_valid_test_datasets_provider, model_provider, forward_step_func=forward_step,
             args_defaults={"tokenizer_type": "NullTokenizer"})
