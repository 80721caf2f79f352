/* onn_b200_host.h -- C driver ABI of libonn_b200_host.so, the C++ host mirror of OpenNN's
 * NeuralNetwork / Transformer / CrossEntropyError3d / AdaptiveMomentEstimation interfaces
 * (opennn_b200/host/opennn_b200.h).  It lets a C, Python (ctypes) or other FFI caller build
 * a network and run the body of OpenNN's training loop
 * (opennn/adaptive_moment_estimation.cpp:697-718: zero gradients, forward_propagate,
 * Loss::back_propagate, update_parameters) on device-resident or host-resident batches.
 *
 * All functions return 0 on success and a negative code on failure;
 * onn_trainer_last_error() then describes it (the C++ layer throws runtime_error exactly
 * where OpenNN does; this ABI catches it at the boundary).
 */
#ifndef ONN_B200_HOST_H
#define ONN_B200_HOST_H

#include <stddef.h>
#include <stdint.h>

#include "onn_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct onn_trainer onn_trainer;

#define ONN_NETWORK_TRANSFORMER   0   /* Transformer (opennn/standard_networks.cpp:638-907) */
#define ONN_NETWORK_DECODER_ONLY  1   /* causal self-attention stack assembled with add_layer */

const char* onn_trainer_last_error(void);

/* Builds the network, its propagation structures for `micro_batch` samples, the loss
 * (regularisation "None") and Adam (lr 1e-3, betas 0.9 / 0.999, clip norm 1, iteration 1).
 * A step processes its batch in chunks of micro_batch samples and accumulates gradients,
 * so device memory is sized by micro_batch, not by the batch. */
int onn_trainer_create(onn_trainer** out, int network_kind,
                       int64_t input_sequence_length, int64_t decoder_sequence_length,
                       int64_t input_vocabulary_size, int64_t output_vocabulary_size,
                       int64_t embedding_dimension, int64_t heads_number,
                       int64_t feed_forward_dimension, int64_t layers_number, int64_t micro_batch);
void onn_trainer_destroy(onn_trainer* trainer);

int64_t onn_trainer_parameters_number(const onn_trainer* trainer);
int onn_trainer_layers_number(const onn_trainer* trainer);
/* name = OpenNN layer type ("Embedding", "MultiHeadAttention", "Addition3d", "Normalization3d",
 * "Dense3d"), label = e.g. "encoder_self_attention_1"; buffers of `capacity` bytes each. */
int onn_trainer_layer_info(const onn_trainer* trainer, int layer, char* name, char* label, int capacity,
                           int64_t* parameters, int64_t* output_size);

/* NeuralNetwork::copy_parameters_device / copy_parameters_host; the arena layout is OpenNN's. */
int onn_trainer_set_parameters(onn_trainer* trainer, const float* host_parameters);
int onn_trainer_get_parameters(onn_trainer* trainer, float* host_parameters);
int onn_trainer_get_gradients(onn_trainer* trainer, float* host_gradients);
int onn_trainer_set_learning_rate(onn_trainer* trainer, float learning_rate);
int onn_trainer_set_iteration(onn_trainer* trainer, int64_t iteration);

/* Data parallelism: every rank holds a full replica and calls step with its shard of the
 * batch; gradients and the active-token count are summed across ranks (onn_dp_*).
 * A step that updates reduce-scatters the gradient arena bucket by bucket from inside back-propagation, runs the
 * norm, clip and Adam on this rank's 1/world of every bucket (the moments exist for that share only) and all-gathers
 * the updated parameters; a step with update = 0 all-reduces, so that every rank can read the whole gradient.
 * onn_trainer_set_dp_options, BEFORE onn_trainer_set_dp: sharded_update = 0 keeps the all-reduce and the whole update
 * on every rank (ONN_B200_DP_SHARDED=0 does the same); carve_sms > 0 makes the persistent kernels of the carve_launches
 * launches that follow a bucket (rounded up to a layer) leave that many SMs free for NCCL's kernels
 * (ONN_B200_DP_CARVE_SMS, ONN_B200_DP_CARVE_LAUNCHES; see onn_set_sm_limit); bucket_floats > 0 sets the size of a
 * gradient bucket (default 16 Mi floats = 64 MiB, ONN_B200_DP_BUCKET_FLOATS).
 * world = 1 (comm NULL) returns the trainer to single-GPU steps; moments are not carried over between the two modes.
 * An exception in the middle of a data-parallel step marks the communicator failed (onn_dp_mark_failed). */
int onn_trainer_set_dp(onn_trainer* trainer, onn_dp_comm* comm, int world);
int onn_trainer_set_dp_options(onn_trainer* trainer, int sharded_update, int carve_sms, int carve_launches, int64_t bucket_floats);

/* CUDA-graph replay of the micro-batch (forward, loss, back-propagation), on by default (ONN_B200_GRAPHS=0 or
 * enabled = 0 turns it off).  The first step runs eagerly; after that every micro-batch index is captured once
 * (opennn/adaptive_moment_estimation.cpp:697-721 launches its ~500 kernels one by one every step) and replayed
 * with its ids copied to fixed device buffers.  The data-parallel rank's last micro-batch, whose back-propagation
 * hands gradient buckets to the all-reduce as it goes, always runs eagerly.  Results do not change. */
int onn_trainer_set_graph_capture(onn_trainer* trainer, int enabled);

/* One optimiser step on a batch of `batch` samples (a multiple of micro_batch, at most 64 micro-batches).
 * After back-propagation the step gathers the bounded-wait status words of its kernels in stream order
 * (onn_device_status_gather); the update does not run if one is set, and the call that next synchronises (a step with
 * statistics, onn_trainer_synchronize) or the next step returns ONN_ERR_DEVICE_TIMEOUT.
 * ids and targets are floats holding integers, [batch, sequence]; encoder_ids is NULL for
 * the decoder-only network.  update = 0 stops after back-propagation (gradients stay in the
 * arena for onn_trainer_get_gradients; the next step starts by zeroing them).
 * statistics (host, 4 floats, may be NULL) receives {error, accuracy, active tokens, gradient
 * norm before clipping}; reading it is the step's one device-to-host synchronisation.
 * _device: pointers are device memory.  _host: pointers are host memory (pinned for full
 * copy speed); the host-to-device copies are part of the step. */
int onn_trainer_step_device(onn_trainer* trainer, const float* decoder_ids, const float* encoder_ids, const float* targets,
                            int64_t batch, int update, float* statistics);
int onn_trainer_step_host(onn_trainer* trainer, const float* decoder_ids, const float* encoder_ids, const float* targets,
                          int64_t batch, int update, float* statistics);
/* The same step fed with 32-bit integer ids in (pinned) host memory, as a data feed holds them
 * (opennn/dataset.cpp:4363-4494 converts to float on the host and copies on the compute path).  The copies go through
 * a copy stream into one of two sets of device buffers, so with statistics = NULL the next call's ids cross PCIe
 * while this call's step computes; the conversion to the floats the layers read is a kernel on the trainer's stream. */
int onn_trainer_step_host_i32(onn_trainer* trainer, const int32_t* decoder_ids, const int32_t* encoder_ids, const int32_t* targets,
                              int64_t batch, int update, float* statistics);

/* NeuralNetwork::forward_propagate on one micro-batch of device-resident ids
 * (is_training = 0: the output layer holds probabilities). */
int onn_trainer_forward(onn_trainer* trainer, const float* decoder_ids, const float* encoder_ids, int is_training);
/* Greedy decoding on token ids: the loop of Transformer::calculate_outputs (opennn/standard_networks.cpp:1002-1035)
 * without the tokeniser and vocabulary maps around it.  encoder_ids (host, [micro_batch, input_sequence_length]) are
 * decoded independently row by row; decoded_ids (host, [micro_batch, decoder_sequence_length]) receives
 * [start_id, token 1, ..., end_id, PAD ...].  The encoder side runs once, the decoder side once per token, the
 * arg-max stays on the device (onn_greedy_next_token); there is no key/value cache. */
int onn_trainer_greedy_decode(onn_trainer* trainer, const float* encoder_ids, float* decoded_ids, int start_id, int end_id);
/* The same decoding with cached keys and values: the encoder side runs once, every decoder-side layer then sees ONE
 * target position per token ([micro_batch, 1, features]); self-attention layers append that position's key and value
 * rows to a cache and attend over it (onn_decode_attention), cross-attention layers attend over keys and values
 * projected once from the encoder output.  Work per token is O(length) instead of O(length^2). */
int onn_trainer_greedy_decode_cached(onn_trainer* trainer, const float* encoder_ids, float* decoded_ids, int start_id, int end_id);
int onn_trainer_get_layer_output(onn_trainer* trainer, int layer, float* host_output, int64_t count);
int onn_trainer_synchronize(onn_trainer* trainer);
/* After a data-parallel step with the sharded update the all-gathers that bring the other ranks' updated parameters
 * are still running: the next step's forward pass waits for them layer by layer, and every entry point of this header
 * that reads or writes parameters waits for all of them first (onn_trainer_synchronize included).  A caller that
 * launches its OWN work on onn_trainer_stream() against the parameter arena, or that times steps with events on that
 * stream, calls this first: it makes the stream wait for the gathers in flight (no host synchronisation).
 * ONN_B200_DP_DEFER_GATHER=0 makes every step wait for its own gathers instead. */
int onn_trainer_parameters_ready(onn_trainer* trainer);
/* Phase tracing: with it on (or ONN_B200_TRACE_PHASES=1) a step records events on the trainer's stream at its start,
 * after the forward pass of its last micro-batch, after that micro-batch's back-propagation and after the update;
 * onn_trainer_last_step_phases synchronises the stream and returns the three intervals in milliseconds
 * {start -> forward done (earlier micro-batches included), back-propagation, update}.  The last micro-batch must
 * have run eagerly (a data-parallel rank's always does; otherwise onn_trainer_set_graph_capture(t, 0)). */
/* Graph segments the data-parallel rank's exchanging micro-batch is replayed from (it cannot be one graph: between its
 * kernels the host enqueues collectives and waits for marks of the communication stream, so it is cut there and the
 * host acts between the segments); 0 = that micro-batch runs kernel by kernel (not recorded yet, graphs off, phase
 * tracing or SM carving on, or the recording failed). */
int onn_trainer_exchange_segments(const onn_trainer* trainer);
int onn_trainer_trace_phases(onn_trainer* trainer, int enabled);
int onn_trainer_last_step_phases(onn_trainer* trainer, float* milliseconds3);
/* The cudaStream_t every kernel of this trainer is launched on (for event timing by the caller). */
void* onn_trainer_stream(onn_trainer* trainer);

/* -------------------------------------------------------------------------------------
 * Text classification (opennn/standard_networks.cpp:575-615, TextClassificationNetwork): Embedding (scaled, with
 * positions) -> self-attention -> max Pooling3d over the sequence -> Dense<2> "RectifiedLinear" layers ->
 * Dense<2> "Softmax" (one class: Dense<2> "Sigmoid"), trained with CrossEntropyError2d
 * (opennn/cross_entropy_error.cpp:58-77, 114-134; one class: the binary form, :36-55, 90-110) and Adam
 * (lr 1e-3, betas 0.9 / 0.999, clip norm 1, iteration 1).  One GPU, one batch per step of exactly `batch` samples.
 * ids [batch, sequence_length] (token ids as floats, 0 = padding) and targets [batch, classes] (one-hot) are DEVICE
 * pointers (one class: targets [batch, 1] holding 0 or 1).  statistics (host, 2 floats, optional) receives {error, gradient norm}.
 * ------------------------------------------------------------------------------------- */
typedef struct onn_classifier onn_classifier;
const char* onn_classifier_last_error(void);
int onn_classifier_create(onn_classifier** out, int64_t vocabulary_size, int64_t sequence_length, int64_t embedding_dimension,
                          int64_t heads_number, const int64_t* hidden_sizes, int hidden_layers, int64_t classes, int64_t batch);
void onn_classifier_destroy(onn_classifier* classifier);
int64_t onn_classifier_parameters_number(const onn_classifier* classifier);
int onn_classifier_layers_number(const onn_classifier* classifier);
int onn_classifier_layer_info(const onn_classifier* classifier, int layer, char* name, char* label, int capacity, int64_t* parameters);
int onn_classifier_set_parameters(onn_classifier* classifier, const float* host_parameters);
int onn_classifier_get_parameters(onn_classifier* classifier, float* host_parameters);
int onn_classifier_get_gradients(onn_classifier* classifier, float* host_gradients);
int onn_classifier_set_learning_rate(onn_classifier* classifier, float learning_rate);
/* calculate_outputs: probabilities [batch, classes] to the host (optional) */
int onn_classifier_forward(onn_classifier* classifier, const float* ids, float* host_probabilities);
/* forward pass, loss, back-propagation and (update != 0) the Adam update */
int onn_classifier_step_device(onn_classifier* classifier, const float* ids, const float* targets, int update, float* statistics);
/* Output of one layer after the last forward pass (for parity checks), and its size in floats. */
int onn_classifier_get_layer_output(onn_classifier* classifier, int layer, float* host_output, int64_t count);
int64_t onn_classifier_layer_output_size(const onn_classifier* classifier, int layer);
/* Data-parallel training: every rank steps its own `batch` samples; the gradient arena and {error, samples} are
 * summed over the ranks after back-propagation (onn_dp_allreduce) and the update divides by the rank count, since the
 * loss is a mean over samples.  onn_classifier_get_gradients then returns the sum over ranks.  world = 1: off. */
int onn_classifier_set_dp(onn_classifier* classifier, onn_dp_comm* comm, int world);

#ifdef __cplusplus
}
#endif

#endif /* ONN_B200_HOST_H */
