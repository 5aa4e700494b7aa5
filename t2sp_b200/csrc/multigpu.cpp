// Sharding of the contractions over the GPUs of one box, for C and C++ hosts: one process (or host
// thread) per GPU, every rank calls the same entry with its rank and the world size.
//
// The reference is single-device (its runtime opens devices[0] only,
// t2s/src/AOT-OpenCL-Runtime.cpp:186-213), so nothing here replaces reference code; the entries keep
// the reference's calling convention (halide_buffer_t in, halide error code out). Every operator has an
// independent output dimension, so ranks work on disjoint output slabs from disjoint or replicated
// inputs and the contractions themselves need no collective:
//
//   GEMM     columns j of B and C          (A replicated)
//   conv     batch items n of I and O      (weights replicated)
//   capsule  batch items n of P and V      (weights replicated)
//   TTM      index j of a(l,i,j), c(i,j,k) (b replicated)
//   MTTKRP   index k of a(l,i,k), b(k,r)   (the contraction): every rank gets a full-size partial d
//
// A slab is the same memory with a shifted base address and unchanged strides, which a
// halide_buffer_t (and the TMA descriptor made from it) describes as it is: shards are views, never
// copies. The exchange steps are separate calls over NCCL, for callers that want the result on every
// GPU: the column gather of a sharded GEMM and the sum of the MTTKRP partials. NCCL is looked up at
// run time (libnccl.so.2) on the first collective call, so single-GPU hosts need not have it.
#include <dlfcn.h>
#include <nccl.h>
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <vector>

#include "host_rt.h"

using namespace t2sp;

namespace {

struct Nccl {
    bool tried = false, ok = false;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};
Nccl g_nccl;
std::mutex g_nccl_mu;

const Nccl* nccl() {
    std::lock_guard<std::mutex> lk(g_nccl_mu);
    if (!g_nccl.tried) {
        g_nccl.tried = true;
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) {
            fprintf(stderr, "t2sp_b200: NCCL is not available (%s); the collective entries need libnccl.so.2\n", dlerror());
            return nullptr;
        }
#define T2SP_SYM(field, name) \
    g_nccl.field = reinterpret_cast<decltype(g_nccl.field)>(dlsym(h, name)); \
    if (!g_nccl.field) { fprintf(stderr, "t2sp_b200: libnccl lacks %s\n", name); return nullptr; }
        T2SP_SYM(GetUniqueId, "ncclGetUniqueId")
        T2SP_SYM(CommInitRank, "ncclCommInitRank")
        T2SP_SYM(CommDestroy, "ncclCommDestroy")
        T2SP_SYM(AllGather, "ncclAllGather")
        T2SP_SYM(AllReduce, "ncclAllReduce")
        T2SP_SYM(Broadcast, "ncclBroadcast")
        T2SP_SYM(GetErrorString, "ncclGetErrorString")
#undef T2SP_SYM
        g_nccl.ok = true;
    }
    return g_nccl.ok ? &g_nccl : nullptr;
}

int nccl_fail(const Nccl* n, const char* what, ncclResult_t r) {
    fprintf(stderr, "t2sp_b200: %s failed: %s\n", what, n->GetErrorString(r));
    return halide_error_code_device_run_failed;
}

int bad_world(int rank, int world) {
    if (world >= 1 && rank >= 0 && rank < world) return 0;
    fprintf(stderr, "t2sp_b200: rank %d is not inside a world of %d\n", rank, world);
    return halide_error_code_constraint_violated;
}

size_t elem_bytes(const halide_buffer_t* b) { return (b->type.bits + 7) / 8; }

// One operand of a sharded call: the caller's buffer or a slab view of it with dimensions of its own.
struct View {
    halide_buffer_t buf;
    halide_dimension_t dims[16];
    halide_buffer_t* src = nullptr;
    halide_buffer_t* get() { return &buf; }
    // what the call changed in the view's state belongs to the caller's buffer too
    void publish() {
        if (!src) return;
        src->flags |= buf.flags & 3u;
    }
};

}  // namespace

extern "C" {

void t2sp_b200_split_range(int64_t total, int32_t world, int32_t rank, int64_t* lo, int64_t* hi) {
    // contiguous and near-equal: the first total % world ranks get one element more
    if (world < 1) world = 1;
    const int64_t base = total / world, extra = total % world;
    const int64_t l = rank * base + (rank < extra ? rank : extra);
    if (lo) *lo = l;
    if (hi) *hi = l + base + (rank < extra ? 1 : 0);
}

int t2sp_b200_shard_view(const halide_buffer_t* src, int32_t dim, int32_t unit, int32_t rank, int32_t world,
                         halide_buffer_t* dst, halide_dimension_t* dst_dims) {
    if (!src || !dst || !dst_dims) return halide_error_code_buffer_argument_is_null;
    if (int e = bad_world(rank, world)) return e;
    if (dim < 0 || dim >= src->dimensions || unit < 1 || src->dim[dim].extent % unit) {
        fprintf(stderr, "t2sp_b200: cannot shard dimension %d (extent %d) in units of %d\n", dim,
                dim >= 0 && dim < src->dimensions ? src->dim[dim].extent : -1, unit);
        return halide_error_code_constraint_violated;
    }
    int64_t lo, hi;
    t2sp_b200_split_range(src->dim[dim].extent / unit, world, rank, &lo, &hi);
    *dst = *src;
    for (int d = 0; d < src->dimensions; ++d) dst_dims[d] = src->dim[d];
    dst->dim = dst_dims;
    dst_dims[dim].extent = static_cast<int32_t>((hi - lo) * unit);
    // `host` and `device` address the element at the buffer's mins: the slab starts lo * unit elements further on
    const int64_t shift = lo * unit * int64_t(src->dim[dim].stride) * int64_t(elem_bytes(src));
    if (dst->host) dst->host += shift;
    if (dst->device) dst->device += shift;
    return 0;
}

}  // extern "C"

namespace {

int make_view(View& v, halide_buffer_t* src, int dim, int unit, int rank, int world) {
    if (!src) return halide_error_code_buffer_argument_is_null;
    if (buf_is_bounds_query(src)) {
        fprintf(stderr, "t2sp_b200: a sharded call needs real buffers (bounds queries are answered by the unsharded entry)\n");
        return halide_error_code_host_is_null;
    }
    if (src->dimensions > 16) return halide_error_code_bad_dimensions;
    v.src = src;
    return t2sp_b200_shard_view(src, dim, unit, rank, world, &v.buf, v.dims);
}

}  // namespace

extern "C" {

int t2sp_b200_gemm_shard(halide_buffer_t* A, halide_buffer_t* B, halide_buffer_t* C, const t2sp_gemm_desc* desc,
                         int32_t rank, int32_t world) {
    if (!A || !B || !C) return halide_error_code_buffer_argument_is_null;
    if ((desc && desc->layout) || C->dimensions != 2) {
        fprintf(stderr, "t2sp_b200_gemm_shard: the column sharding applies to the plain 2-D output layout\n");
        return halide_error_code_constraint_violated;
    }
    if (B->dimensions != 2) return halide_error_code_bad_dimensions;
    View b, c;
    const int jdim = (desc && desc->trans_b) ? 1 : 0;  // where the column index j lives in B
    if (int e = make_view(b, B, jdim, 1, rank, world)) return e;
    if (int e = make_view(c, C, 0, 1, rank, world)) return e;
    const int rc = t2sp_b200_gemm(A, b.get(), c.get(), desc);
    b.publish();
    c.publish();
    return rc;
}

int t2sp_b200_conv_shard(halide_buffer_t* I, halide_buffer_t* K, halide_buffer_t* O, const t2sp_conv_desc* desc,
                         int32_t rank, int32_t world) {
    if (!I || !K || !O || !desc) return halide_error_code_buffer_argument_is_null;
    if (desc->layout || desc->CI < 1 || desc->CO < 1) {
        fprintf(stderr, "t2sp_b200_conv_shard: the batch sharding applies to the plain 2-D output layout\n");
        return halide_error_code_constraint_violated;
    }
    View i, o;  // dimension 0 is (channel + channels * n): whole images, CI resp. CO elements each
    if (int e = make_view(i, I, 0, desc->CI, rank, world)) return e;
    if (int e = make_view(o, O, 0, desc->CO, rank, world)) return e;
    const int rc = t2sp_b200_conv(i.get(), K, o.get(), desc);
    i.publish();
    o.publish();
    return rc;
}

int t2sp_b200_capsule_shard(halide_buffer_t* P, halide_buffer_t* W, halide_buffer_t* V, const t2sp_capsule_desc* desc,
                            int32_t rank, int32_t world) {
    if (!P || !W || !V || !desc) return halide_error_code_buffer_argument_is_null;
    if (desc->layout || (desc->stride != 1 && desc->stride != 2)) {
        fprintf(stderr, "t2sp_b200_capsule_shard: the batch sharding applies to the plain 2-D output layout\n");
        return halide_error_code_constraint_violated;
    }
    const int s = desc->stride;
    const int IY = s * desc->OY + desc->KY - s, IX = s * desc->OX + desc->KX - s;
    View p, v;  // dimension 1 is (pixel + pixels * n)
    if (int e = make_view(p, P, 1, IY * IX, rank, world)) return e;
    if (int e = make_view(v, V, 1, desc->OY * desc->OX, rank, world)) return e;
    const int rc = t2sp_b200_capsule(p.get(), W, v.get(), desc);
    p.publish();
    v.publish();
    return rc;
}

int t2sp_b200_ttm_shard(halide_buffer_t* a, halide_buffer_t* b, halide_buffer_t* c, const t2sp_ttm_desc* desc,
                        int32_t rank, int32_t world) {
    if (!a || !b || !c) return halide_error_code_buffer_argument_is_null;
    if ((desc && desc->layout) || c->dimensions != 3 || a->dimensions != 3) {
        fprintf(stderr, "t2sp_b200_ttm_shard: the j sharding applies to the plain 3-D output layout\n");
        return halide_error_code_constraint_violated;
    }
    View av, cv;
    if (int e = make_view(av, a, 2, 1, rank, world)) return e;
    if (int e = make_view(cv, c, 1, 1, rank, world)) return e;
    const int rc = t2sp_b200_ttm(av.get(), b, cv.get(), desc);
    av.publish();
    cv.publish();
    return rc;
}

int t2sp_b200_mttkrp_shard(halide_buffer_t* a, halide_buffer_t* b, halide_buffer_t* c, halide_buffer_t* d_partial,
                           const t2sp_mttkrp_desc* desc, int32_t rank, int32_t world) {
    if (!a || !b || !c || !d_partial) return halide_error_code_buffer_argument_is_null;
    if (a->dimensions != 3 || b->dimensions != 2) return halide_error_code_bad_dimensions;
    View av, bv;
    if (int e = make_view(av, a, 2, 1, rank, world)) return e;
    if (int e = make_view(bv, b, 0, 1, rank, world)) return e;
    const int rc = t2sp_b200_mttkrp(av.get(), bv.get(), c, d_partial, desc);
    av.publish();
    bv.publish();
    return rc;
}

// ------------------------------------------------------------------------------ collectives (NCCL)
int t2sp_b200_nccl_unique_id(void* id_bytes, int32_t size) {
    const Nccl* n = nccl();
    if (!n) return halide_error_code_device_interface_no_device;
    if (!id_bytes || size < static_cast<int32_t>(sizeof(ncclUniqueId))) return halide_error_code_buffer_argument_is_null;
    ncclUniqueId id;
    if (ncclResult_t r = n->GetUniqueId(&id)) return nccl_fail(n, "ncclGetUniqueId", r);
    memcpy(id_bytes, &id, sizeof(id));
    return 0;
}

int t2sp_b200_comm_init(void** comm, int32_t world, const void* id_bytes, int32_t rank) {
    const Nccl* n = nccl();
    if (!n) return halide_error_code_device_interface_no_device;
    if (!comm || !id_bytes) return halide_error_code_buffer_argument_is_null;
    if (int e = bad_world(rank, world)) return e;
    if (int e = rt_ensure_device()) return e;  // makes the calling thread's device current
    ncclUniqueId id;
    memcpy(&id, id_bytes, sizeof(id));
    ncclComm_t c = nullptr;
    if (ncclResult_t r = n->CommInitRank(&c, world, id, rank)) return nccl_fail(n, "ncclCommInitRank", r);
    *comm = c;
    return 0;
}

int t2sp_b200_comm_destroy(void* comm) {
    const Nccl* n = nccl();
    if (!n) return halide_error_code_device_interface_no_device;
    if (!comm) return 0;
    if (ncclResult_t r = n->CommDestroy(static_cast<ncclComm_t>(comm))) return nccl_fail(n, "ncclCommDestroy", r);
    return 0;
}

int t2sp_b200_broadcast(halide_buffer_t* buf, void* comm, int32_t root) {
    const Nccl* n = nccl();
    if (!n) return halide_error_code_device_interface_no_device;
    if (!buf || !comm) return halide_error_code_buffer_argument_is_null;
    if (!buf_on_our_device(buf)) return halide_error_code_no_device_interface;
    if (int e = rt_ensure_device()) return e;
    const size_t bytes = static_cast<size_t>(buf_elems_span(buf)) * elem_bytes(buf);
    void* p = reinterpret_cast<void*>(buf->device);
    if (ncclResult_t r = n->Broadcast(p, p, bytes, ncclChar, root, static_cast<ncclComm_t>(comm), rt_stream()))
        return nccl_fail(n, "ncclBroadcast", r);
    buf->flags |= 2u;
    buf->flags &= ~uint64_t(1);
    return tls().async ? 0 : rt_check_status("broadcast");
}

int t2sp_b200_gather_columns(halide_buffer_t* C, void* comm, int32_t rank, int32_t world) {
    const Nccl* n = nccl();
    if (!n) return halide_error_code_device_interface_no_device;
    if (!C || !comm) return halide_error_code_buffer_argument_is_null;
    if (int e = bad_world(rank, world)) return e;
    if (C->dimensions != 2 || C->dim[0].stride != 1) return halide_error_code_bad_dimensions;
    if (!buf_on_our_device(C)) {
        fprintf(stderr, "t2sp_b200_gather_columns: C must be resident on the device (t2sp_b200_device_malloc or wrap_device_ptr)\n");
        return halide_error_code_no_device_interface;
    }
    if (int e = rt_ensure_device()) return e;
    const int64_t N = C->dim[0].extent, M = C->dim[1].extent, ld = C->dim[1].stride;
    const size_t es = elem_bytes(C);
    if (N == 0 || M == 0 || world == 1) return 0;
    // NCCL gathers equal contiguous pieces; a column slab is neither, so it goes through staging:
    // pack this rank's slab, all-gather, unpack the other ranks' slabs into their columns of C.
    int64_t lo, hi;
    t2sp_b200_split_range(N, world, 0, &lo, &hi);
    const int64_t wmax = hi - lo;  // rank 0's slab is among the widest
    const size_t piece = size_t(M) * wmax * es;
    char* send = static_cast<char*>(rt_alloc(piece));
    char* recv = static_cast<char*>(rt_alloc(piece * world));
    if (!send || !recv) {
        rt_free(send);
        rt_free(recv);
        return halide_error_code_device_malloc_failed;
    }
    cudaStream_t s = rt_stream();
    char* base = reinterpret_cast<char*>(C->device);
    t2sp_b200_split_range(N, world, rank, &lo, &hi);
    bool ok = true;
    if (hi > lo)
        ok &= cudaMemcpy2DAsync(send, wmax * es, base + lo * es, ld * es, (hi - lo) * es, M, cudaMemcpyDeviceToDevice, s) == cudaSuccess;
    ncclResult_t r = ok ? n->AllGather(send, recv, piece, ncclChar, static_cast<ncclComm_t>(comm), s) : ncclSuccess;
    for (int g = 0; ok && r == ncclSuccess && g < world; ++g) {
        if (g == rank) continue;
        t2sp_b200_split_range(N, world, g, &lo, &hi);
        if (hi > lo)
            ok &= cudaMemcpy2DAsync(base + lo * es, ld * es, recv + piece * g, wmax * es, (hi - lo) * es, M,
                                    cudaMemcpyDeviceToDevice, s) == cudaSuccess;
    }
    rt_free(send);
    rt_free(recv);
    if (r != ncclSuccess) return nccl_fail(n, "ncclAllGather", r);
    if (!ok) {
        cudaGetLastError();
        return halide_error_code_device_buffer_copy_failed;
    }
    C->flags |= 2u;
    return tls().async ? 0 : rt_check_status("gather_columns");
}

int t2sp_b200_reduce_partials(halide_buffer_t* d, void* comm, int32_t rank, int32_t world, int32_t ordered) {
    const Nccl* n = nccl();
    if (!n) return halide_error_code_device_interface_no_device;
    if (!d || !comm) return halide_error_code_buffer_argument_is_null;
    if (int e = bad_world(rank, world)) return e;
    if (d->dimensions != 2 || d->dim[0].stride != 1 || d->type.bits != 32) return halide_error_code_bad_dimensions;
    if (!buf_on_our_device(d)) return halide_error_code_no_device_interface;
    if (int e = rt_ensure_device()) return e;
    const int I = d->dim[0].extent, R = d->dim[1].extent;
    const int64_t ld = d->dim[1].stride;
    if (I == 0 || R == 0 || world == 1) return 0;
    cudaStream_t s = rt_stream();
    float* pd = reinterpret_cast<float*>(d->device);
    if (!ordered && ld == I) {
        if (ncclResult_t r = n->AllReduce(pd, pd, size_t(I) * R, ncclFloat, ncclSum, static_cast<ncclComm_t>(comm), s))
            return nccl_fail(n, "ncclAllReduce", r);
        return tls().async ? 0 : rt_check_status("reduce_partials");
    }
    // Reproducible form: gather every rank's partial and add them in rank order, the same ordered sum
    // the split-K kernels end with (the result does not depend on a reduction tree).
    const size_t piece = size_t(I) * R * sizeof(float);
    float* send = static_cast<float*>(rt_alloc(piece));
    float* recv = static_cast<float*>(rt_alloc(piece * world));
    if (!send || !recv) {
        rt_free(send);
        rt_free(recv);
        return halide_error_code_device_malloc_failed;
    }
    bool ok = cudaMemcpy2DAsync(send, size_t(I) * 4, pd, ld * 4, size_t(I) * 4, R, cudaMemcpyDeviceToDevice, s) == cudaSuccess;
    ncclResult_t r = ok ? n->AllGather(send, recv, piece, ncclChar, static_cast<ncclComm_t>(comm), s) : ncclSuccess;
    if (ok && r == ncclSuccess) {
        ok = reduce_partials_launch(recv, pd, I, R, ld, world, s) == cudaSuccess;
        rt_count_launch(1);
    }
    rt_free(send);
    rt_free(recv);
    if (r != ncclSuccess) return nccl_fail(n, "ncclAllGather", r);
    if (!ok) {
        cudaGetLastError();
        return halide_error_code_device_run_failed;
    }
    d->flags |= 2u;
    return tls().async ? 0 : rt_check_status("reduce_partials");
}

}  // extern "C"
