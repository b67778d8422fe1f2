"""LeNet-style CNN for 3x32x32 images (the shape of CIFAR-10), used by the DDP example and the
CPU fault-injection tests.  Same architecture as the example model in the reference's
``train_ddp.py:91-108``: conv 3->6 (5x5), pool, conv 6->16 (5x5), pool, fc 400->120->84->10."""

import torch
from torch import nn


class LeNet(nn.Module):
    def __init__(self, num_classes: int = 10) -> None:
        super().__init__()
        self.features = nn.Sequential(
            nn.Conv2d(3, 6, 5),
            nn.ReLU(),
            nn.MaxPool2d(2, 2),
            nn.Conv2d(6, 16, 5),
            nn.ReLU(),
            nn.MaxPool2d(2, 2),
        )
        self.classifier = nn.Sequential(
            nn.Linear(16 * 5 * 5, 120),
            nn.ReLU(),
            nn.Linear(120, 84),
            nn.ReLU(),
            nn.Linear(84, num_classes),
        )

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self.features(x)
        return self.classifier(torch.flatten(x, 1))
