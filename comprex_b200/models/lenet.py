"""LeNet models.

``LeNet5`` is the classic network of the LeNet-5 data-parallel configuration:
conv 6@5x5 -> maxpool 2 -> conv 16@5x5 -> maxpool 2 -> FC 120 -> 84 -> 10 with
ReLU, valid convolutions on 28x28x1 inputs (44 426 parameters).
``LeNetReference`` is the variant the reference trains (LeNet/model.py:9-55):
conv 20@5x5 same -> ReLU -> maxpool 2 -> conv 50@5x5 same -> ReLU -> maxpool 2
-> global average pool -> dense 10 (26 080 parameters).
"""
import torch
import torch.nn as nn
import torch.nn.functional as F


class LeNet5(nn.Module):
    def __init__(self, num_classes: int = 10):
        super().__init__()
        self.conv1 = nn.Conv2d(1, 6, 5)
        self.conv2 = nn.Conv2d(6, 16, 5)
        self.fc1 = nn.Linear(16 * 4 * 4, 120)
        self.fc2 = nn.Linear(120, 84)
        self.fc3 = nn.Linear(84, num_classes)

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.conv1(x)), 2)
        x = F.max_pool2d(F.relu(self.conv2(x)), 2)
        x = torch.flatten(x, 1)
        x = F.relu(self.fc1(x))
        x = F.relu(self.fc2(x))
        return self.fc3(x)


class LeNetReference(nn.Module):
    def __init__(self, num_classes: int = 10):
        super().__init__()
        self.conv1 = nn.Conv2d(1, 20, 5, padding=2)
        self.conv2 = nn.Conv2d(20, 50, 5, padding=2)
        self.fc = nn.Linear(50, num_classes)

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.conv1(x)), 2)
        x = F.max_pool2d(F.relu(self.conv2(x)), 2)
        x = x.mean(dim=(2, 3))
        return self.fc(x)
