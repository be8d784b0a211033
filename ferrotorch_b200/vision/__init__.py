"""Vision: model zoo, detection/box operators, datasets, image IO and transforms (API names follow ferrotorch-vision)."""
from . import models, ops
from .models import (BasicBlock, Bottleneck, ResNet, resnet18, resnet34, resnet50, resnet50_dilated, VGG, vgg11, vgg16, VisionTransformer, vit_b_16,
                     MobileNetV2, mobilenet_v2, DenseNet, densenet121, ConvNeXt, convnext_tiny, EfficientNet, efficientnet_b0, UNet, Yolo,
                     ModelRegistry, ModelConstructor, list_models, get_model, register_model, create_feature_extractor, FeatureExtractor, Conv1x1)
from .ops import (box_convert, box_area, box_iou, generalized_box_iou, distance_box_iou, complete_box_iou, clip_boxes_to_image, remove_small_boxes,
                  nms, batched_nms, sigmoid_focal_loss, focal_loss, roi_align, roi_align_with_aligned, roi_pool)
from .data import (read_image, write_image, Mnist, Cifar10, Cifar100, DatasetFolder, ImageFolder, Compose, ToTensor, VisionNormalize, Resize,
                   CenterCrop, RandomCrop, RandomHorizontalFlip, RandomVerticalFlip, RandomResizedCrop, RandomRotation, ColorJitter, GaussianNoise,
                   RandomGaussianBlur, RandomApply, RandomChoice, ElasticTransform, TrivialAugmentWide, VisionToTensor, vision_manual_seed, RawImage,
                   read_image_raw, read_image_rgba, read_image_as_tensor, raw_image_to_tensor, tensor_to_raw_image, write_raw_image, write_tensor_as_image,
                   Split, MnistSample, CifarSample, IMAGENET_MEAN, IMAGENET_STD)
from . import models2, segmentation, detection  # noqa: E402
from .models2 import MobileNetV3, MobileNetV3Small, MobileNetV3Large, mobilenet_v3_small, mobilenet_v3_large, InceptionV3, inception_v3, SwinTransformer, swin_tiny  # noqa: E402
from .segmentation import Fcn, DeepLabV3, Lraspp, Aspp, FcnHead, DeepLabV3Head, ResNet50Dilated, fcn_resnet50, deeplabv3_resnet50, lraspp_mobilenet_v3_large  # noqa: E402
from .detection import (Detections, MaskDetections, SsdDetections, RpnConfig, RpnHead, TwoMlpHead, MaskHead, MaskPredictor, FPN_OUT_CHANNELS, SSD_ANCHORS_PER_SCALE,
                        SSD_FM_SIZES, SSD_TOTAL_ANCHORS, FeaturePyramidNetwork, AnchorGenerator, Rpn, decode_boxes, encode_boxes, postprocess_detections, postprocess_masks, FasterRcnn,  # noqa: E402
                        MaskRcnn, KeypointRcnn, RetinaNet, Fcos, Ssd300, fasterrcnn_resnet50_fpn, maskrcnn_resnet50_fpn, keypointrcnn_resnet50_fpn,
                        retinanet_resnet50_fpn, fcos_resnet50_fpn, ssd300_vgg16)

for _n, _c in (("mobilenet_v3_small", mobilenet_v3_small), ("mobilenet_v3_large", mobilenet_v3_large), ("inception_v3", inception_v3), ("swin_tiny", swin_tiny),
               ("fcn_resnet50", fcn_resnet50), ("deeplabv3_resnet50", deeplabv3_resnet50), ("lraspp_mobilenet_v3_large", lraspp_mobilenet_v3_large),
               ("fasterrcnn_resnet50_fpn", fasterrcnn_resnet50_fpn), ("maskrcnn_resnet50_fpn", maskrcnn_resnet50_fpn),
               ("keypointrcnn_resnet50_fpn", keypointrcnn_resnet50_fpn), ("retinanet_resnet50_fpn", retinanet_resnet50_fpn), ("fcos_resnet50_fpn", fcos_resnet50_fpn),
               ("ssd300_vgg16", ssd300_vgg16)):
    models.register_model(_n, _c)
