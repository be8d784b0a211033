"""Vision: model zoo, detection/box operators, datasets, image IO and transforms (API names follow ferrotorch-vision)."""
from . import models, ops
from .models import (BasicBlock, Bottleneck, ResNet, resnet18, resnet34, resnet50, resnet50_dilated, VGG, vgg11, vgg16, VisionTransformer, vit_b_16,
                     MobileNetV2, mobilenet_v2, DenseNet, densenet121, ConvNeXt, convnext_tiny, EfficientNet, efficientnet_b0, UNet, Yolo,
                     ModelRegistry, list_models, get_model, register_model, create_feature_extractor, Conv1x1)
from .ops import (box_convert, box_area, box_iou, generalized_box_iou, distance_box_iou, complete_box_iou, clip_boxes_to_image, remove_small_boxes,
                  nms, batched_nms, sigmoid_focal_loss, focal_loss, roi_align, roi_pool)
from .data import (read_image, write_image, Mnist, Cifar10, Cifar100, DatasetFolder, ImageFolder, Compose, ToTensor, VisionNormalize, Resize,
                   CenterCrop, RandomCrop, RandomHorizontalFlip, RandomVerticalFlip, RandomResizedCrop, RandomRotation, ColorJitter, GaussianNoise,
                   RandomGaussianBlur, RandomApply, ElasticTransform, TrivialAugmentWide)
