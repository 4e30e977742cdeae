// The part of the InfiniBand verbs ABI (rdma-core's infiniband/verbs.h) that the verbs transport touches, declared
// locally because the header is not installed on the build image.  The library itself is opened with dlopen at run
// time, like the reference does (csrc/plugins/rdma_executor/utils/rdma_utils.cc:13-53, 23 symbols by dlsym); the
// data-path calls (post_send, post_recv, poll_cq, req_notify_cq) are not exported symbols but function pointers in
// the context's operations table, which is why the layout of ibv_context matters and is spelled out here.
// Only fields that the transport reads or writes are named for what they are; the rest keeps the layout.
#pragma once
#include <pthread.h>
#include <stddef.h>
#include <stdint.h>

extern "C" {

union ibv_gid {
  uint8_t raw[16];
  struct { uint64_t subnet_prefix, interface_id; } global;
};

struct ibv_device;
struct ibv_context;
struct ibv_comp_channel;
struct ibv_srq;
struct ibv_ah;
struct ibv_mw;
struct ibv_qp;
struct ibv_cq;
struct ibv_wc;
struct ibv_send_wr;
struct ibv_recv_wr;

struct ibv_context_ops {
  void* compat_query_device;
  void* compat_query_port;
  void* compat_alloc_pd;
  void* compat_dealloc_pd;
  void* compat_reg_mr;
  void* compat_rereg_mr;
  void* compat_dereg_mr;
  void* alloc_mw;
  void* bind_mw;
  void* dealloc_mw;
  void* compat_create_cq;
  int (*poll_cq)(ibv_cq* cq, int num_entries, ibv_wc* wc);
  int (*req_notify_cq)(ibv_cq* cq, int solicited_only);
  void* compat_cq_event;
  void* compat_resize_cq;
  void* compat_destroy_cq;
  void* compat_create_srq;
  void* compat_modify_srq;
  void* compat_query_srq;
  void* compat_destroy_srq;
  void* post_srq_recv;
  void* compat_create_qp;
  void* compat_query_qp;
  void* compat_modify_qp;
  void* compat_destroy_qp;
  int (*post_send)(ibv_qp* qp, ibv_send_wr* wr, ibv_send_wr** bad_wr);
  int (*post_recv)(ibv_qp* qp, ibv_recv_wr* wr, ibv_recv_wr** bad_wr);
  void* compat_attach_mcast;
  void* compat_detach_mcast;
  void* compat_async_event;
};

struct ibv_context {
  ibv_device* device;
  ibv_context_ops ops;
  int cmd_fd;
  int async_fd;
  int num_comp_vectors;
  pthread_mutex_t mutex;
  void* abi_compat;
};

struct ibv_pd {
  ibv_context* context;
  uint32_t handle;
};

struct ibv_mr {
  ibv_context* context;
  ibv_pd* pd;
  void* addr;
  size_t length;
  uint32_t handle;
  uint32_t lkey;
  uint32_t rkey;
};

struct ibv_cq {
  ibv_context* context;
  ibv_comp_channel* channel;
  void* cq_context;
  uint32_t handle;
  int cqe;
  pthread_mutex_t mutex;
  pthread_cond_t cond;
  uint32_t comp_events_completed;
  uint32_t async_events_completed;
};

enum ibv_qp_state { IBV_QPS_RESET = 0, IBV_QPS_INIT = 1, IBV_QPS_RTR = 2, IBV_QPS_RTS = 3, IBV_QPS_SQD = 4, IBV_QPS_SQE = 5, IBV_QPS_ERR = 6 };
enum ibv_qp_type { IBV_QPT_RC = 2, IBV_QPT_UC = 3, IBV_QPT_UD = 4 };
enum ibv_mtu { IBV_MTU_256 = 1, IBV_MTU_512 = 2, IBV_MTU_1024 = 3, IBV_MTU_2048 = 4, IBV_MTU_4096 = 5 };
enum ibv_mig_state { IBV_MIG_MIGRATED = 0, IBV_MIG_REARM = 1, IBV_MIG_ARMED = 2 };

struct ibv_qp {
  ibv_context* context;
  void* qp_context;
  ibv_pd* pd;
  ibv_cq* send_cq;
  ibv_cq* recv_cq;
  ibv_srq* srq;
  uint32_t handle;
  uint32_t qp_num;
  ibv_qp_state state;
  ibv_qp_type qp_type;
  pthread_mutex_t mutex;
  pthread_cond_t cond;
  uint32_t events_completed;
};

enum ibv_wc_status { IBV_WC_SUCCESS = 0 };
struct ibv_wc {
  uint64_t wr_id;
  int status;
  int opcode;
  uint32_t vendor_err;
  uint32_t byte_len;
  uint32_t imm_data;
  uint32_t qp_num;
  uint32_t src_qp;
  unsigned int wc_flags;
  uint16_t pkey_index;
  uint16_t slid;
  uint8_t sl;
  uint8_t dlid_path_bits;
};

struct ibv_sge {
  uint64_t addr;
  uint32_t length;
  uint32_t lkey;
};

enum ibv_wr_opcode {
  IBV_WR_RDMA_WRITE = 0, IBV_WR_RDMA_WRITE_WITH_IMM = 1, IBV_WR_SEND = 2, IBV_WR_SEND_WITH_IMM = 3, IBV_WR_RDMA_READ = 4,
  IBV_WR_ATOMIC_CMP_AND_SWP = 5, IBV_WR_ATOMIC_FETCH_AND_ADD = 6
};
enum ibv_send_flags { IBV_SEND_FENCE = 1 << 0, IBV_SEND_SIGNALED = 1 << 1, IBV_SEND_SOLICITED = 1 << 2, IBV_SEND_INLINE = 1 << 3 };

struct ibv_mw_bind_info {
  ibv_mr* mr;
  uint64_t addr;
  uint64_t length;
  unsigned int mw_access_flags;
};

struct ibv_send_wr {
  uint64_t wr_id;
  ibv_send_wr* next;
  ibv_sge* sg_list;
  int num_sge;
  int opcode;
  unsigned int send_flags;
  uint32_t imm_data;
  union {
    struct { uint64_t remote_addr; uint32_t rkey; } rdma;
    struct { uint64_t remote_addr; uint64_t compare_add; uint64_t swap; uint32_t rkey; } atomic;
    struct { ibv_ah* ah; uint32_t remote_qpn; uint32_t remote_qkey; } ud;
  } wr;
  union { struct { uint32_t remote_srqn; } xrc; } qp_type;
  union {
    struct { ibv_mw* mw; uint32_t rkey; ibv_mw_bind_info bind_info; } bind_mw;
    struct { void* hdr; uint16_t hdr_sz; uint16_t mss; } tso;
  };
};

struct ibv_qp_cap {
  uint32_t max_send_wr, max_recv_wr, max_send_sge, max_recv_sge, max_inline_data;
};

struct ibv_qp_init_attr {
  void* qp_context;
  ibv_cq* send_cq;
  ibv_cq* recv_cq;
  ibv_srq* srq;
  ibv_qp_cap cap;
  ibv_qp_type qp_type;
  int sq_sig_all;
};

struct ibv_global_route {
  ibv_gid dgid;
  uint32_t flow_label;
  uint8_t sgid_index;
  uint8_t hop_limit;
  uint8_t traffic_class;
};

struct ibv_ah_attr {
  ibv_global_route grh;
  uint16_t dlid;
  uint8_t sl;
  uint8_t src_path_bits;
  uint8_t static_rate;
  uint8_t is_global;
  uint8_t port_num;
};

struct ibv_qp_attr {
  ibv_qp_state qp_state;
  ibv_qp_state cur_qp_state;
  ibv_mtu path_mtu;
  ibv_mig_state path_mig_state;
  uint32_t qkey;
  uint32_t rq_psn;
  uint32_t sq_psn;
  uint32_t dest_qp_num;
  unsigned int qp_access_flags;
  ibv_qp_cap cap;
  ibv_ah_attr ah_attr;
  ibv_ah_attr alt_ah_attr;
  uint16_t pkey_index;
  uint16_t alt_pkey_index;
  uint8_t en_sqd_async_notify;
  uint8_t sq_draining;
  uint8_t max_rd_atomic;
  uint8_t max_dest_rd_atomic;
  uint8_t min_rnr_timer;
  uint8_t port_num;
  uint8_t timeout;
  uint8_t retry_cnt;
  uint8_t rnr_retry;
  uint8_t alt_port_num;
  uint8_t alt_timeout;
  uint32_t rate_limit;
};

enum ibv_qp_attr_mask {
  IBV_QP_STATE = 1 << 0, IBV_QP_CUR_STATE = 1 << 1, IBV_QP_EN_SQD_ASYNC_NOTIFY = 1 << 2, IBV_QP_ACCESS_FLAGS = 1 << 3,
  IBV_QP_PKEY_INDEX = 1 << 4, IBV_QP_PORT = 1 << 5, IBV_QP_QKEY = 1 << 6, IBV_QP_AV = 1 << 7, IBV_QP_PATH_MTU = 1 << 8,
  IBV_QP_TIMEOUT = 1 << 9, IBV_QP_RETRY_CNT = 1 << 10, IBV_QP_RNR_RETRY = 1 << 11, IBV_QP_RQ_PSN = 1 << 12,
  IBV_QP_MAX_QP_RD_ATOMIC = 1 << 13, IBV_QP_ALT_PATH = 1 << 14, IBV_QP_MIN_RNR_TIMER = 1 << 15, IBV_QP_SQ_PSN = 1 << 16,
  IBV_QP_MAX_DEST_RD_ATOMIC = 1 << 17, IBV_QP_PATH_MIG_STATE = 1 << 18, IBV_QP_CAP = 1 << 19, IBV_QP_DEST_QPN = 1 << 20
};

enum ibv_access_flags {
  IBV_ACCESS_LOCAL_WRITE = 1, IBV_ACCESS_REMOTE_WRITE = 1 << 1, IBV_ACCESS_REMOTE_READ = 1 << 2, IBV_ACCESS_REMOTE_ATOMIC = 1 << 3
};

struct ibv_port_attr {
  int state;
  ibv_mtu max_mtu;
  ibv_mtu active_mtu;
  int gid_tbl_len;
  uint32_t port_cap_flags;
  uint32_t max_msg_sz;
  uint32_t bad_pkey_cntr;
  uint32_t qkey_viol_cntr;
  uint16_t pkey_tbl_len;
  uint16_t lid;
  uint16_t sm_lid;
  uint8_t lmc;
  uint8_t max_vl_num;
  uint8_t sm_sl;
  uint8_t subnet_timeout;
  uint8_t init_type_reply;
  uint8_t active_width;
  uint8_t active_speed;
  uint8_t phys_state;
  uint8_t link_layer;
  uint8_t flags;
  uint16_t port_cap_flags2;
  uint32_t active_speed_ex;
};

}  // extern "C"
