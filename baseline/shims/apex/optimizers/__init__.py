"""``FusedSGD`` / ``FusedAdam`` mapped onto PyTorch's own fused CUDA optimizers with apex's keyword
names (``set_grad_none``, ``bias_correction``); apex FusedAdam defaults to decoupled weight decay,
hence AdamW."""
import torch


class FusedSGD(torch.optim.SGD):
    def __init__(self, params, lr=1e-3, momentum=0.0, weight_decay=0.0, set_grad_none=True, **kw):
        super().__init__(params, lr=lr, momentum=momentum, weight_decay=weight_decay,
                         fused=torch.cuda.is_available())


class FusedAdam(torch.optim.AdamW):
    def __init__(self, params, lr=1e-3, eps=1e-8, weight_decay=0.0, bias_correction=True, set_grad_none=True,
                 betas=(0.9, 0.999), **kw):
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                         fused=torch.cuda.is_available())
