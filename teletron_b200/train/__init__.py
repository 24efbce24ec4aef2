from .arguments import build_parser, get_args, get_num_microbatches, parse_args, set_args, validate_args  # noqa: F401
from .microbatches import (BatchSchedule, get_current_global_batch_size,  # noqa: F401
                           update_num_microbatches)
from .trainer import Float16Module, Trainer  # noqa: F401
from .helpers import (calc_params_l2_norm, get_attr_wrapped_model, get_grad_norm,  # noqa: F401
                      get_train_valid_test_num_samples, is_last_rank, num_floating_point_operations,
                      print_datetime, print_rank_0, print_rank_last, report_memory, report_theoretical_memory,
                      update_train_iters)
from .hunyuan_step import make_hunyuan_forward_step  # noqa: F401
from .wan_step import average_losses_across_data_parallel_group, make_forward_step  # noqa: F401
