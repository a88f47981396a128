/*
 * Test stand-in for <ucp/api/ucp.h>: the handful of UCP types, constants and calls that
 * plugins/ucx/plugin.cc uses, with the names and argument order of UCX 1.1x, implemented over
 * TCP sockets in plugins/ucx/fake_ucp.cc.  It exists so that the UCX plugin's own logic
 * (listener queue, endpoints, tagged posts, polling, registration, forced close) can be built and
 * exercised on machines without UCX.  It is not UCX and is never installed.
 */
#ifndef UCCL_FAKE_UCP_API_H_
#define UCCL_FAKE_UCP_API_H_

#include <stddef.h>
#include <stdint.h>
#include <sys/socket.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  UCS_OK = 0,
  UCS_INPROGRESS = 1,
  UCS_ERR_NO_MEMORY = -4,
  UCS_ERR_INVALID_PARAM = -5,
  UCS_ERR_UNREACHABLE = -6,
  UCS_ERR_MESSAGE_TRUNCATED = -9,
  UCS_ERR_CONNECTION_RESET = -25,
  UCS_ERR_LAST = -100
} ucs_status_t;
typedef void* ucs_status_ptr_t;
#define UCS_PTR_IS_ERR(p) (((uintptr_t)(p)) >= ((uintptr_t)UCS_ERR_LAST))
#define UCS_PTR_IS_PTR(p) (((uintptr_t)(p) - 1) < ((uintptr_t)UCS_ERR_LAST - 1))
#define UCS_PTR_STATUS(p) ((ucs_status_t)(intptr_t)(p))
#define UCS_STATUS_PTR(s) ((void*)(intptr_t)(s))
const char* ucs_status_string(ucs_status_t status);

typedef enum { UCS_THREAD_MODE_SINGLE = 0, UCS_THREAD_MODE_SERIALIZED = 1, UCS_THREAD_MODE_MULTI = 2 } ucs_thread_mode_t;
typedef enum { UCS_MEMORY_TYPE_HOST = 0, UCS_MEMORY_TYPE_CUDA = 1 } ucs_memory_type_t;

typedef struct ucp_context* ucp_context_h;
typedef struct ucp_config ucp_config_t;
typedef struct ucp_worker* ucp_worker_h;
typedef struct ucp_listener* ucp_listener_h;
typedef struct ucp_ep* ucp_ep_h;
typedef struct ucp_conn_request* ucp_conn_request_h;
typedef struct ucp_mem* ucp_mem_h;
typedef uint64_t ucp_tag_t;
typedef uint64_t ucp_datatype_t;

enum { UCP_PARAM_FIELD_FEATURES = 1 << 0 };
enum { UCP_FEATURE_TAG = 1 << 0, UCP_FEATURE_RMA = 1 << 1, UCP_FEATURE_STREAM = 1 << 5 };
typedef struct {
  uint64_t field_mask;
  uint64_t features;
} ucp_params_t;

enum { UCP_WORKER_PARAM_FIELD_THREAD_MODE = 1 << 0 };
typedef struct {
  uint64_t field_mask;
  ucs_thread_mode_t thread_mode;
} ucp_worker_params_t;

typedef struct {
  const struct sockaddr* addr;
  socklen_t addrlen;
} ucs_sock_addr_t;
typedef void (*ucp_listener_conn_callback_t)(ucp_conn_request_h conn_request, void* arg);
typedef struct {
  ucp_listener_conn_callback_t cb;
  void* arg;
} ucp_listener_conn_handler_t;
enum { UCP_LISTENER_PARAM_FIELD_SOCK_ADDR = 1 << 0, UCP_LISTENER_PARAM_FIELD_CONN_HANDLER = 1 << 2 };
typedef struct {
  uint64_t field_mask;
  ucs_sock_addr_t sockaddr;
  ucp_listener_conn_handler_t conn_handler;
} ucp_listener_params_t;
enum { UCP_LISTENER_ATTR_FIELD_SOCKADDR = 1 << 0 };
typedef struct {
  uint64_t field_mask;
  struct sockaddr_storage sockaddr;
} ucp_listener_attr_t;

typedef enum { UCP_ERR_HANDLING_MODE_NONE = 0, UCP_ERR_HANDLING_MODE_PEER = 1 } ucp_err_handling_mode_t;
enum {
  UCP_EP_PARAM_FIELD_ERR_HANDLING_MODE = 1 << 1,
  UCP_EP_PARAM_FIELD_SOCK_ADDR = 1 << 4,
  UCP_EP_PARAM_FIELD_FLAGS = 1 << 5,
  UCP_EP_PARAM_FIELD_CONN_REQUEST = 1 << 6
};
enum { UCP_EP_PARAMS_FLAGS_CLIENT_SERVER = 1 << 0 };
typedef struct {
  uint64_t field_mask;
  ucp_err_handling_mode_t err_mode;
  unsigned flags;
  ucs_sock_addr_t sockaddr;
  ucp_conn_request_h conn_request;
} ucp_ep_params_t;

enum { UCP_OP_ATTR_FIELD_FLAGS = 1 << 5 };
enum { UCP_EP_CLOSE_FLAG_FORCE = 1 << 0 };
typedef struct {
  uint32_t op_attr_mask;
  uint32_t flags;
  void* request;
  void* user_data;
  ucp_datatype_t datatype;
} ucp_request_param_t;
typedef struct {
  ucp_tag_t sender_tag;
  size_t length;
} ucp_tag_recv_info_t;

enum {
  UCP_MEM_MAP_PARAM_FIELD_ADDRESS = 1 << 0,
  UCP_MEM_MAP_PARAM_FIELD_LENGTH = 1 << 1,
  UCP_MEM_MAP_PARAM_FIELD_MEMORY_TYPE = 1 << 4
};
typedef struct {
  uint64_t field_mask;
  void* address;
  size_t length;
  unsigned flags;
  ucs_memory_type_t memory_type;
} ucp_mem_map_params_t;

ucs_status_t ucp_config_read(const char* env_prefix, const char* filename, ucp_config_t** config_p);
void ucp_config_release(ucp_config_t* config);
ucs_status_t ucp_init(const ucp_params_t* params, const ucp_config_t* config, ucp_context_h* context_p);
void ucp_cleanup(ucp_context_h context);
ucs_status_t ucp_worker_create(ucp_context_h context, const ucp_worker_params_t* params, ucp_worker_h* worker_p);
void ucp_worker_destroy(ucp_worker_h worker);
unsigned ucp_worker_progress(ucp_worker_h worker);
ucs_status_t ucp_listener_create(ucp_worker_h worker, const ucp_listener_params_t* params, ucp_listener_h* listener_p);
ucs_status_t ucp_listener_query(ucp_listener_h listener, ucp_listener_attr_t* attr);
void ucp_listener_destroy(ucp_listener_h listener);
ucs_status_t ucp_ep_create(ucp_worker_h worker, const ucp_ep_params_t* params, ucp_ep_h* ep_p);
ucs_status_ptr_t ucp_ep_close_nbx(ucp_ep_h ep, const ucp_request_param_t* param);
ucs_status_ptr_t ucp_tag_send_nbx(ucp_ep_h ep, const void* buffer, size_t count, ucp_tag_t tag, const ucp_request_param_t* param);
ucs_status_ptr_t ucp_tag_recv_nbx(ucp_worker_h worker, void* buffer, size_t count, ucp_tag_t tag, ucp_tag_t tag_mask,
                                  const ucp_request_param_t* param);
ucs_status_t ucp_request_check_status(void* request);
ucs_status_t ucp_tag_recv_request_test(void* request, ucp_tag_recv_info_t* info);
void ucp_request_free(void* request);
ucs_status_t ucp_mem_map(ucp_context_h context, const ucp_mem_map_params_t* params, ucp_mem_h* memh_p);
ucs_status_t ucp_mem_unmap(ucp_context_h context, ucp_mem_h memh);

/* test hook of the stand-in: registrations alive right now (leak check) */
int fake_ucp_live_registrations(void);

#ifdef __cplusplus
}
#endif
#endif
