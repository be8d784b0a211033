// Host-side detection primitives: greedy non-maximum suppression over score-sorted boxes (O(kept * N) time, O(N) memory).
// Capability parity: ferrotorch-vision/src/ops.rs:209 (nms), :279 (batched_nms).
#include <cstdint>
#include <vector>

#define FT_EXPORT extern "C" __attribute__((visibility("default")))

// boxes: [n, 4] (x0, y0, x1, y1) already sorted by decreasing score. keep[i] = 1 if box i survives. Returns the number kept.
FT_EXPORT int64_t ft_nms_sorted_f32(const float* boxes, int64_t n, float iou_threshold, uint8_t* keep) {
  std::vector<float> area((size_t)n);
  for (int64_t i = 0; i < n; i++) {
    const float* b = boxes + 4 * i;
    area[(size_t)i] = (b[2] - b[0]) * (b[3] - b[1]);
    keep[i] = 1;
  }
  int64_t kept = 0;
  for (int64_t i = 0; i < n; i++) {
    if (!keep[i]) continue;
    kept++;
    const float* a = boxes + 4 * i;
    for (int64_t j = i + 1; j < n; j++) {
      if (!keep[j]) continue;
      const float* b = boxes + 4 * j;
      const float xx0 = a[0] > b[0] ? a[0] : b[0], yy0 = a[1] > b[1] ? a[1] : b[1];
      const float xx1 = a[2] < b[2] ? a[2] : b[2], yy1 = a[3] < b[3] ? a[3] : b[3];
      const float w = xx1 - xx0 > 0.f ? xx1 - xx0 : 0.f, h = yy1 - yy0 > 0.f ? yy1 - yy0 : 0.f;
      const float inter = w * h;
      if (inter / (area[(size_t)i] + area[(size_t)j] - inter) > iou_threshold) keep[j] = 0;
    }
  }
  return kept;
}
