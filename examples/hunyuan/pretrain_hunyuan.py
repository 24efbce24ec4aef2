"""HunyuanVideo pre-training entry point: ``torchrun ... examples/hunyuan/pretrain_hunyuan.py <flags>``.

Same contract as the Wan example: ``Trainer(parse_args(extra_args)).pretrain(forward_step)`` with the
library's HunyuanVideo flow-matching step (teletron_b200.train.make_hunyuan_forward_step).  With
``--distributed-vae`` the batches come from encoder ranks in the schema ``prompt_embeds, clip_text_embed,
first_ref_image, latents``; with ``--synthetic-latents`` they are generated locally.
"""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from teletron_b200.train import Trainer, make_hunyuan_forward_step, parse_args  # noqa: E402


def extra_args(parser):
    group = parser.add_argument_group(title="hunyuan args")
    group.add_argument("--num-single-layers", type=int, default=None)
    group.add_argument("--num-refiner-layers", type=int, default=None)
    group.add_argument("--text-embed-dim", type=int, default=None)
    group.add_argument("--pooled-projection-dim", type=int, default=None)
    group.add_argument("--text-len", type=int, default=256)
    group.add_argument("--embedded-guidance", type=float, default=6.0)
    group.add_argument("--encoder-name", type=str, default=None)
    return parser


if __name__ == "__main__":
    args = parse_args(extra_args=extra_args)
    trainer = Trainer(args)
    trainer.pretrain(forward_step_func=make_hunyuan_forward_step(
        shift=args.flow_shift if args.flow_shift != 5.0 else 7.0, train_timesteps=args.flow_train_timesteps,
        embedded_guidance=args.embedded_guidance))
