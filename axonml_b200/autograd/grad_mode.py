"""Thread-local gradient modes (crates/axonml-autograd/src/no_grad.rs:133-220)."""
import torch

no_grad = torch.no_grad
enable_grad = torch.enable_grad
inference_mode = torch.inference_mode
set_grad_enabled_context = torch.set_grad_enabled
is_grad_enabled = torch.is_grad_enabled
is_inference_mode = torch.is_inference_mode_enabled
