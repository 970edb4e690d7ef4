"""Multi-model ("dist-train") jobs: sub-models on disjoint rank ranges, and depth-parallel 3-D convolution."""
from .dist_train import (DistTrainConfig, SubModelConfig, get_dist_model_config, get_dist_model_index, initialize_dist_train,
                         is_in_model, recv_from_previous_model, send_to_next_model, send_grad_to_previous_model,
                         recv_grad_from_next_model, dist_forward_backward, destroy_dist_train)
from .conv3d_depth_parallel import Conv3dDepthParallel

__all__ = ["DistTrainConfig", "SubModelConfig", "initialize_dist_train", "get_dist_model_config", "get_dist_model_index",
           "is_in_model", "send_to_next_model", "recv_from_previous_model", "send_grad_to_previous_model",
           "recv_grad_from_next_model", "dist_forward_backward", "destroy_dist_train", "Conv3dDepthParallel"]
