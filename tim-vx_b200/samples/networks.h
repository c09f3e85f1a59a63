/*
 * Seeded synthetic networks built through the public tim::vx API only, with a
 * small C interface so that tests and the benchmark can drive them from
 * Python.  They play the role of the reference's samples (samples/lenet,
 * samples/multi_device/vx_resnet50.cc, vx_mobilenet.cc), whose trained weight
 * files are not available: shapes and op sequences are the published
 * architectures, weights and inputs are random with a fixed seed.
 *
 *   "lenet"        LeNet-5 as in samples/lenet/lenet_asymu8.cc:115-290; uint8 weights zp 128
 *   "resnet50"     ResNet-50 v1.5, uint8 activations, per-channel int8 weights
 *   "mobilenetv2"  MobileNetV2-1.0, uint8 activations and uint8 weights (zero point in [100,156],
 *                  values drawn symmetrically about it so that each channel sums to zero)
 */
#ifndef B2VX_SAMPLES_NETWORKS_H_
#define B2VX_SAMPLES_NETWORKS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b2vx_net b2vx_net;

/* Builds and compiles the network; NULL on failure (reason on stderr). */
b2vx_net* b2vx_net_create(const char* name, int32_t batch, uint64_t seed, int32_t device);
void b2vx_net_destroy(b2vx_net* net);
size_t b2vx_net_input_bytes(const b2vx_net* net);   /* uint8 [W,H,C,batch] */
size_t b2vx_net_output_bytes(const b2vx_net* net);  /* uint8 [classes,batch] */
/* Fills `dst` with the seeded synthetic input of this network (uniform 0..255). */
void b2vx_net_synthetic_input(const b2vx_net* net, uint64_t seed, uint8_t* dst);
/* Tensor::CopyDataToTensor / Graph::Run / Tensor::CopyDataFromTensor; 0 on success. */
int32_t b2vx_net_set_input(b2vx_net* net, const void* data);
int32_t b2vx_net_run(b2vx_net* net);
int32_t b2vx_net_get_output(b2vx_net* net, void* data);
/* The b2vx_graph behind the tim::vx graph, for launch-plan readback and profiling. */
void* b2vx_net_graph_handle(b2vx_net* net);
/* MACs and algorithmic activation+weight bytes of one image, as built. */
uint64_t b2vx_net_macs_per_image(const b2vx_net* net);

#ifdef __cplusplus
}
#endif
#endif /* B2VX_SAMPLES_NETWORKS_H_ */
