"""Model zoo: the CIFAR architectures of the research harness (selected by name, as
paper-code/tasks/cifar.py:167 does), the LSTM language model, GPT-2 and the small MLP."""
from .densenet import DenseNet121, DenseNet161, DenseNet169, DenseNet201, densenet_cifar  # noqa: F401
from .dpn import DPN26, DPN92  # noqa: F401
from .googlenet import GoogLeNet  # noqa: F401
from .gpt2 import GPT2, GPT2Config  # noqa: F401
from .lenet import LeNet  # noqa: F401
from .lstm import RNNModel, wikitext2_lstm  # noqa: F401
from .mlp import MLP  # noqa: F401
from .mobilenet import MobileNet, MobileNetV2  # noqa: F401
from .pnasnet import PNASNetA, PNASNetB  # noqa: F401
from .preact_resnet import PreActResNet18, PreActResNet34, PreActResNet50, PreActResNet101, PreActResNet152  # noqa: F401
from .resnet import ResNet18, ResNet34, ResNet50, ResNet101, ResNet152  # noqa: F401
from .resnext import ResNeXt29_2x64d, ResNeXt29_4x64d, ResNeXt29_8x64d, ResNeXt29_32x4d  # noqa: F401
from .senet import SENet18  # noqa: F401
from .shufflenet import ShuffleNetG2, ShuffleNetG3  # noqa: F401
from .vgg import vgg11, vgg11_bn, vgg13, vgg13_bn, vgg16, vgg16_bn, vgg19, vgg19_bn  # noqa: F401
